// bfloat16 attention for prompt portions on the 5th-generation tensor cores (tcgen05), keys
// and values read from the paged cache.
//
// One block owns 256 rows = 2 x (128 / G) consecutive tokens of one sequence x the G query
// heads of one key/value head, as TWO query tiles of 128 rows (a token's G heads in G
// consecutive rows; the last 128 % G rows of a tile stay empty), A (the earlier tokens) and B,
// and walks the keys in tiles of 128.  Every key and
// value tile is brought into shared memory once and used by both query tiles: a block reads
// half the cache bytes per product that a block of 128 rows would, and it is the traffic from
// L2 into the SMs (every block of rows re-reads the keys it sees) that bounds this kernel at
// long contexts.  For each query tile g and key tile t:
//   S_g = Q_g . K^T  one 128 x 128 x head_dim product into tensor memory (tcgen05.mma, operands in
//                    shared memory, both K-major, 128-byte swizzle)
//   softmax          eight warps in TWO GROUPS of 128 threads, group g on query tile g, one thread
//                    per row: the running maximum and sum of a row need no shuffles and nothing is
//                    exchanged between threads.  A thread reads its row's 128 scores twice
//                    (tcgen05.ld): once for the maximum, once for exp2 on pre-scaled scores in
//                    32-bit (packed f32x2 FMA/ADD and the 3-input max of sm_100 keep the
//                    instruction count down); the probabilities go BACK INTO TENSOR MEMORY as
//                    bfloat16 (tcgen05.st), over the scores they were made from
//   O_g += P_g . V   one 128 x head_dim x 128 product with P read from tensor memory; V's tile is
//                    used as it lies in the pages (head_dim contiguous: an MN-major operand), O_g
//                    stays in tensor memory (S_A, S_B, O_A, O_B: 4 x 128 columns, all there is)
// The scores of a query tile have one stage; the overlap comes from the two query tiles: while
// group A works on its probabilities the tensor cores compute P_B . V and the next Q_B . K, and
// the other way round.  P takes no shared memory, which leaves room for three stages of K and
// two of V beside the two query tiles.
// A row's output is rescaled only when its maximum grew by more than 2^8 (the stale maximum
// keeps every probability below 256, harmless in bfloat16 and float32); then the row's
// thread reads, scales and writes back its row of O_g (tcgen05.ld / tcgen05.st).
// A ninth warp allocates tensor memory and issues the MMAs; two more bring
// the key and the value tiles in with TMA, one box of 64 columns x page_size rows per page and
// half of head_dim, straight from the paged cache (no cluster multicast), as soon as a stage
// is free.  Pages the block table does not name are skipped; the stages are zeroed once, so
// such rows hold finite values that the masks then exclude.  A block whose sequence ends within
// its first 128 rows (the end of a prompt, a single decoded token of a mixed batch) runs
// query tile A alone; tile A also leaves out a last key tile that only tile B's tokens see.
// Every wait on an mbarrier is bounded; a wait that runs out raises the block's abort flag,
// which ends all roles, and the status word reports it.
//
// Formula and masking: spymaster2h/spyinfer src/backends/cpu/cpu_attention.cpp:89-135.  The
// reference's prefill kernel (src/backends/cuda/native/attention.cu:62-255) uses no tensor
// cores and cannot see a cached prefix.
// Limits (checked on the host): head_dim 64 or 128, G <= 16, bfloat16, a page size of 8, 16,
// 32, 64 or 128 tokens (a page is one TMA box and must tile the 128-key tile).
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

SPY_MODULE(spy_attention_tc)

namespace {

using namespace tc;

constexpr int ROWS = 128;            // rows of a query tile = UMMA M
constexpr int BLOCK_ROWS = 2 * ROWS; // query rows per block: tiles A and B
constexpr int TILE = 128;            // keys per tile = UMMA N of the first product
constexpr int K_STAGES = 3;          // K tiles in flight
constexpr int V_STAGES = 2;          // V tiles in flight
constexpr int SOFTMAX_THREADS = 256; // warps 0..7: Q load, softmax (two groups of 128, a thread per row), epilogue
constexpr int GROUP_THREADS = 128;
constexpr int NUM_THREADS = 352;     // warp 8: TMEM + MMA; warps 9, 10: TMA of K and of V
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;

struct Params {
    const bf16* q;
    long long q_stride;
    bf16* out;                 // [T, nh * hd]
    const int* block_table;    // [S, table_width]
    const int* positions;      // [T]
    const int* q_start;        // [S + 1]
    int* status;
    int table_width, page_size, num_pages, nh, nkv, G, Gp, S, window;
    int hd;                    // the head size as stored (a multiple of 8, at most HD): the tiles are HD wide, what lies beyond hd is zero
    int x_blocks, items;       // 256-row blocks along the tokens (an upper bound), and x_blocks * nkv work items
    float scale_log2;
};

// One work item: 256 query rows of one sequence and key/value head, and the key tiles they see.
// tiles_a, tiles_b: key tiles that query tile A / B works on, counted from tile_first (tiles_b = 0: the sequence
// ends within tile A); n_tiles = the larger of the two = the key tiles that are loaded.
struct Item {
    int seq, tok0, kvh, n_tiles, tile_first, block_lo, block_last_pos, tok_end;
    int tiles_a, tiles_b;
};

// Byte offset of 16-byte chunk `chunk` (0 .. HD / 8 - 1) of row `row` in a [128 rows][64-element halves]
// tile with 128-byte swizzle.
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk)
{
    return (uint32_t)((chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int HD> struct Smem {
    static constexpr int OPERAND_BYTES = ROWS * HD * 2;       // a Q, K or V tile
    static constexpr int Q_OFF = 0;                                  // query tiles A and B
    static constexpr int K_OFF = Q_OFF + 2 * OPERAND_BYTES;          // K_STAGES stages
    static constexpr int V_OFF = K_OFF + K_STAGES * OPERAND_BYTES;   // V_STAGES stages
    static constexpr int BAR_OFF = V_OFF + V_STAGES * OPERAND_BYTES;
    // barriers, the tensor-memory slot, the abort flag and the two work items: 320 bytes.  The dynamic shared memory is
    // declared with an alignment of 1024 bytes (what the 128-byte swizzle needs), so no slack is added to align it by
    // hand; the kernel checks the alignment and reports instead of running if it ever were not so.
    static constexpr int TOTAL = BAR_OFF + 320;
    static constexpr int TMEM_COLS = 512;                     // S_A, S_B: 128 columns each (P over the first 64 of S); O_A, O_B: HD columns each from 256
};

// Pipeline (key tile t of the item; K in stage t % 3, V in stage t % 2 of the running tile number):
//   softmax group g:  wait S_g(t) | read, max | if O_g must be rescaled: wait P_g.V(t-1), rescale | read, exp | write P_g(t) | signal
//   MMA thread:       Q_A.K(0), Q_B.K(0), then for every t:
//                     wait P_A(t), V(t) | P_A.V(t) | wait K(t+1) | Q_A.K(t+1) | wait P_B(t) | P_B.V(t) | Q_B.K(t+1)
// so the tensor cores work on query tile B while group A works on its probabilities, and the other way round.
template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, 1) attention_tc_kernel(const __grid_constant__ CUtensorMap page_map, const Params p)
{
    using L = Smem<HD>;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    uint8_t* smem = smem_raw;
    if ((smem_u32(smem) & 1023u) != 0) {   // never seen; without the alignment the tiles' swizzle would not match the descriptors
        if (threadIdx.x == 0) report_status(p.status, SPY_STATUS_WAIT_TIMEOUT, -2);
        return;
    }
    uint64_t* bar_k = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);   // [K_STAGES] K tile landed (TMA bytes)
    uint64_t* bar_v = bar_k + K_STAGES;                                 // [V_STAGES] V tile landed (TMA bytes)
    uint64_t* bar_kfree = bar_v + V_STAGES;                             // [K_STAGES] the last Q.K of the stage's tile is complete (MMA commit)
    uint64_t* bar_vfree = bar_kfree + K_STAGES;                         // [V_STAGES] the last P.V of the stage's tile is complete (MMA commit)
    uint64_t* bar_s = bar_vfree + V_STAGES;                             // [2] a query tile's scores are complete (MMA commit)
    uint64_t* bar_p = bar_s + 2;                                        // [2] its probabilities are written (the group's 128 arrivals)
    uint64_t* bar_o = bar_p + 2;                                        // [2] its P.V is complete (MMA commit)
    uint64_t* bar_epi = bar_o + 2;                                      // [2] its accumulator has been read out at the end of an item in which it had tiles (128 arrivals)
    uint64_t* bar_q = bar_epi + 2;                                      // the item's Q tiles are written (256 arrivals)
    uint64_t* bar_item = bar_q + 1;                                     // [2] the block's next work item is described (thread 0)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_item + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    Item* item_ring = reinterpret_cast<Item*>(tmem_slot + 2);           // [2]

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int tokens_per_tile = ROWS / p.Gp, tokens_per_block = 2 * tokens_per_tile;   // a tile's last ROWS % Gp rows stay empty
    if (tid == 0) {
        for (int i = 0; i < K_STAGES; ++i) {
            mbar_init(bar_k + i, 1);
            mbar_init(bar_kfree + i, 1);
        }
        for (int i = 0; i < V_STAGES; ++i) {
            mbar_init(bar_v + i, 1);
            mbar_init(bar_vfree + i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_s + i, 1);
            mbar_init(bar_p + i, GROUP_THREADS);
            mbar_init(bar_o + i, 1);
            mbar_init(bar_epi + i, GROUP_THREADS);
            mbar_init(bar_item + i, 1);
        }
        mbar_init(bar_q, SOFTMAX_THREADS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(tmem_slot, L::TMEM_COLS);
    // rows of pages the block table does not name are never copied: keep them finite
    for (int i = tid; i < (K_STAGES + V_STAGES) * L::OPERAND_BYTES / 16; i += NUM_THREADS) reinterpret_cast<uint4*>(smem + L::K_OFF)[i] = make_uint4(0, 0, 0, 0);
    fence_async_proxy();
    pdl_wait();   // everything below reads what earlier kernels wrote

    // The block's work items.  The items are numbered with the long ones first (in a causal prompt the
    // late rows see the most keys): item i is the block of rows x_blocks - 1 - i / nkv, counted through
    // the sequences, of key/value head i % nkv.  The block takes one item a round, forwards in even rounds
    // and backwards in odd ones, so that a long item of one round meets a short one of the next.
    const int G_blocks = (int)gridDim.x, blk = (int)blockIdx.x;
    auto item_index = [&](int k) { return k * G_blocks + ((k & 1) ? G_blocks - 1 - blk : blk); };
    // Thread 0 describes the block's (j + 1)-th item WITH TILES while the block works on the j-th; every role
    // waits for the description.  Rounds whose item has no tiles (x_blocks is an upper bound) are passed over
    // here, so that every entry of the ring is real work: thread 0 can then never be two entries ahead of a
    // role that has not read its entry yet.  After the last item an entry with n_tiles = -1 ends the roles.
    int next_round = 0;   // thread 0 only
    auto describe_next = [&](int j) {
        Item it;
        it.seq = -1; it.tok0 = 0; it.kvh = 0; it.n_tiles = -1; it.tile_first = 0; it.block_lo = 0; it.block_last_pos = -1; it.tok_end = 0;
        it.tiles_a = it.tiles_b = 0;
        for (; it.n_tiles <= 0; ++next_round) {
            const int i = item_index(next_round);
            if (i >= p.items) { it.n_tiles = -1; break; }
            it.kvh = i % p.nkv;
            it.seq = -1;
            int b = p.x_blocks - 1 - i / p.nkv;
            for (int s = 0; s < p.S; ++s) {
                const int n = p.q_start[s + 1] - p.q_start[s];
                const int blocks = (n + tokens_per_block - 1) / tokens_per_block;
                if (b < blocks) { it.seq = s; it.tok0 = p.q_start[s] + b * tokens_per_block; break; }
                b -= blocks;
            }
            if (it.seq < 0) continue;
            it.tok_end = p.q_start[it.seq + 1];
            const int first_pos = p.positions[it.tok0];
            it.block_last_pos = p.positions[min(it.tok_end, it.tok0 + tokens_per_block) - 1];
            const int a_last_pos = p.positions[min(it.tok_end, it.tok0 + tokens_per_tile) - 1];
            it.block_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
            if (it.block_lo <= it.block_last_pos) {
                it.tile_first = it.block_lo / TILE;
                it.n_tiles = it.block_last_pos / TILE - it.tile_first + 1;
                it.tiles_a = a_last_pos / TILE - it.tile_first + 1;                          // at least one: block_lo <= first_pos <= a_last_pos
                it.tiles_b = it.tok0 + tokens_per_tile < it.tok_end ? it.n_tiles : 0;
            }
        }
        item_ring[j & 1] = it;
        mbar_arrive(bar_item + (j & 1));   // releases the description to the waiting roles
    };
    if (tid == 0) describe_next(0);
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 2 * TILE;
    const uint32_t q_s = smem_u32(smem + L::Q_OFF), k_s = smem_u32(smem + L::K_OFF), v_s = smem_u32(smem + L::V_OFF);
    // Every role walks the same entries j = 0, 1, ... and counts the same tiles: `base` key tiles before the
    // current item's (the stages and phases of K and V follow base + t), and for each query tile the tiles it
    // has worked on (the phases of its scores, probabilities and products follow that count).

    if (warp < 8) {
        // ---------------------------------------------------------------- loads, softmax, epilogue
        const int row = tid & (ROWS - 1), grp = tid >> 7;     // this thread's row of its query tile = TMEM lane, and its group = the query tile
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        constexpr int HALF = TILE / 2;       // scores read at a time
        const uint32_t tmem_s = tmem_base + grp * TILE + lane_addr;   // the group's scores and probabilities, this thread's row
        const uint32_t tmem_og = tmem_o + grp * HD + lane_addr;       // the group's accumulator, this thread's row
        bool alive = true, q_requested = false;
        int count = 0;                       // tiles this group has worked on
        // The group's Q tile: consecutive threads copy consecutive 16-byte pieces of a row.  It is requested as soon
        // as the group's last product of the item before is complete (every Q.K of that query tile is then complete),
        // and so arrives while that item's output is read and stored.
        auto request_q = [&](const Item& it) {
            constexpr int CPR = HD / 8;
            if ((grp == 0 ? it.tiles_a : it.tiles_b) <= 0) return;
            for (int idx = row; idx < ROWS * CPR; idx += GROUP_THREADS) {
                const int r = idx / CPR, c = idx % CPR;
                const int r_tok = it.tok0 + grp * tokens_per_tile + r / p.Gp, r_hg = r % p.Gp;
                const bool ok = r / p.Gp < tokens_per_tile && r_tok < it.tok_end && r_hg < p.G && c * 8 < p.hd;   // rows and columns beyond the data are filled with zeros
                const bf16* src = p.q + (size_t)(ok ? r_tok : 0) * p.q_stride + (size_t)(it.kvh * p.G + (ok ? r_hg : 0)) * p.hd + (ok ? c * 8 : 0);
                cp_async16(smem + L::Q_OFF + grp * L::OPERAND_BYTES + tile_offset(r, c), src, ok);
            }
        };
        for (int j = 0; alive; ++j) {
            alive = mbar_wait(bar_item + (j & 1), (uint32_t)(j >> 1) & 1, abort_flag);
            if (!alive) break;
            const Item it = item_ring[j & 1];
            if (it.n_tiles < 0) break;
            const int my_tiles = grp == 0 ? it.tiles_a : it.tiles_b, tile_first = it.tile_first, tok_end = it.tok_end, kvh = it.kvh;
            const int tok = it.tok0 + grp * tokens_per_tile + row / p.Gp, hg = row % p.Gp;
            const bool row_ok = row / p.Gp < tokens_per_tile && tok < tok_end && hg < p.G;
            const int head = kvh * p.G + hg;
            // the keys this row sees
            const int pos = row_ok ? min(p.positions[tok], it.block_last_pos) : -1;
            const int lo = max((row_ok && p.window > 0) ? max(0, p.positions[tok] - p.window + 1) : 0, it.block_lo);
            if (!q_requested) request_q(it);   // the block's first item
            asm volatile("cp.async.wait_all;" ::: "memory");
            fence_async_proxy();   // the MMA reads shared memory through the async proxy
            mbar_arrive(bar_q);
            if (tid == 0) describe_next(j + 1);   // while the first scores are on their way

            float m_used = -INFINITY, l = 0.f;   // the maximum the row's probabilities are taken against, and their sum
            for (int t = 0; t < my_tiles; ++t, ++count) {
                const uint32_t ph = (uint32_t)count & 1;
                alive = mbar_wait(bar_s + grp, ph, abort_flag);          // S_g(t) is complete
                if (!alive) break;
                fence_after_sync();
                const int key0 = (tile_first + t) * TILE;
                const bool whole = __all_sync(0xffffffffu, !row_ok || (key0 >= lo && key0 + TILE - 1 <= pos));
                // First reading of the row's 128 raw scores: the maximum, by 3-input max in four independent chains
                // (on the raw scores: the scale is positive).  Scores the row does not see count as -inf.
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t sc[HALF];
#pragma unroll
                    for (int c = 0; c < HALF; c += 32) tmem_load<32>(tmem_s + h * HALF + c, *reinterpret_cast<uint32_t(*)[32]>(&sc[c]));
                    tmem_wait_ld();
                    if (!whole) {
#pragma unroll
                        for (int i = 0; i < HALF; ++i) {
                            const int k = key0 + h * HALF + i;
                            if (!(k <= pos && k >= lo)) sc[i] = 0xff800000u;   // -inf
                        }
                    }
#pragma unroll
                    for (int i = 0; i < HALF; i += 8) {
#pragma unroll
                        for (int c = 0; c < 4; ++c) mx4[c] = max3(mx4[c], __uint_as_float(sc[i + 2 * c]), __uint_as_float(sc[i + 2 * c + 1]));
                    }
                }
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
                // the maximum in use moves only when the row's maximum grew by more than the threshold (or from nothing)
                const float m_new = fmaxf(m_used, mx);
                const bool grow = m_new > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && m_new != -INFINITY);
                const float alpha = grow ? (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new)) : 1.f;
                if (grow) {
                    l *= alpha;
                    m_used = m_new;
                }
                // Only a rescale of the accumulator has to wait for the tile's last product, so in the common case
                // P_g(t) is ready before the tensor core asks for it.  The item's first tile overwrites the accumulator.
                if (t > 0 && __any_sync(0xffffffffu, grow)) {
                    alive = mbar_wait(bar_o + grp, (uint32_t)(count - 1) & 1, abort_flag);
                    if (!alive) break;
                    fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t r[32];
                        tmem_load<32>(tmem_og + c, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_store<32>(tmem_og + c, r);
                        tmem_wait_st();
                    }
                }
                // Second reading: the probabilities.  The scale is folded into the exponent's argument,
                // exp2(s * scale - m), one packed FMA for two scores; the sum runs in two packed accumulators.  P goes
                // over the first 64 columns of S, 64 keys at a time: the columns written have been read before.
                const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
                const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), neg2 = pack2(neg_m, neg_m);
                uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    uint32_t sc[HALF];
#pragma unroll
                    for (int c = 0; c < HALF; c += 32) tmem_load<32>(tmem_s + h * HALF + c, *reinterpret_cast<uint32_t(*)[32]>(&sc[c]));
                    tmem_wait_ld();
                    if (!whole) {
#pragma unroll
                        for (int i = 0; i < HALF; ++i) {
                            const int k = key0 + h * HALF + i;
                            if (!(k <= pos && k >= lo)) sc[i] = 0xff800000u;
                        }
                    }
                    uint32_t packed[HALF / 2];
#pragma unroll
                    for (int i = 0; i < HALF; i += 2) {
                        float a0, a1;
                        unpack2(fma2(pack2(__uint_as_float(sc[i]), __uint_as_float(sc[i + 1])), scale2, neg2), a0, a1);
                        const float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
                        sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], pack2(p0, p1));
                        packed[i / 2] = pack_bf16(p0, p1);
                    }
                    tmem_store<32>(tmem_s + h * (HALF / 2), packed);
                }
                {
                    float s0, s1;
                    unpack2(add2(sum2[0], sum2[1]), s0, s1);
                    l += s0 + s1;
                }
                tmem_wait_st();
                fence_before_sync();
                mbar_arrive(bar_p + grp);
            }
            if (!alive) break;
            // ---- the query tile's last product is complete, and with it (the tensor core runs in order) all of its products
            if (my_tiles > 0) {
                alive = mbar_wait(bar_o + grp, (uint32_t)(count - 1) & 1, abort_flag);
                if (!alive) break;
                fence_after_sync();
            }
            // ---- the next item's Q tile is requested ...
            alive = mbar_wait(bar_item + ((j + 1) & 1), (uint32_t)((j + 1) >> 1) & 1, abort_flag);
            if (!alive) break;
            q_requested = item_ring[(j + 1) & 1].n_tiles > 0;
            if (q_requested) request_q(item_ring[(j + 1) & 1]);
            // ---- ... and this item's output is read and stored meanwhile: O_g / l
            if (my_tiles > 0) {
                const float inv = l > 0.f ? 1.f / l : 0.f;
                bf16* dst = p.out + ((size_t)(row_ok ? tok : 0) * p.nh + head) * p.hd;
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    uint32_t r[32];
                    tmem_load<32>(tmem_og + c, r);
                    tmem_wait_ld();
                    if (!row_ok) continue;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 v;
                        v.x = pack_bf16(__uint_as_float(r[8 * q4]) * inv, __uint_as_float(r[8 * q4 + 1]) * inv);
                        v.y = pack_bf16(__uint_as_float(r[8 * q4 + 2]) * inv, __uint_as_float(r[8 * q4 + 3]) * inv);
                        v.z = pack_bf16(__uint_as_float(r[8 * q4 + 4]) * inv, __uint_as_float(r[8 * q4 + 5]) * inv);
                        v.w = pack_bf16(__uint_as_float(r[8 * q4 + 6]) * inv, __uint_as_float(r[8 * q4 + 7]) * inv);
                        if (c + 8 * q4 < p.hd) *reinterpret_cast<uint4*>(dst + c + 8 * q4) = v;
                    }
                }
            }
            // the next product into this accumulator overwrites it: the tensor core waits for this.  Only a group that had tiles
            // arrives (and only such items are counted on the other side): a group without tiles runs ahead through the item,
            // and a barrier that completed twice before it was waited on once would never be seen to complete.
            if (my_tiles > 0) {
                fence_before_sync();
                mbar_arrive(bar_epi + grp);
            }
        }
    } else if (warp == 8) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc_qk = instr_desc_bf16(ROWS, TILE, false, false), idesc_pv = instr_desc_bf16(ROWS, HD, false, true);
            auto issue_qk = [&](int g, int gt) {   // query tile g against the key tile with running number gt
                const uint32_t qb = q_s + g * L::OPERAND_BYTES, kb = k_s + (gt % K_STAGES) * L::OPERAND_BYTES;
#pragma unroll
                for (int s = 0; s < HD / 16; ++s) {
                    const uint32_t off = (s >> 2) * (ROWS * 128) + (s & 3) * 32;   // 64-element half, then 32 bytes per 16 elements
                    umma(tmem_base + g * TILE, desc_k_major(qb + off), desc_k_major(kb + off), idesc_qk, s > 0 ? 1u : 0u);
                }
                umma_commit(bar_s + g);
            };
            auto issue_pv = [&](int g, int gt, bool first) {
                const uint32_t vb = v_s + (gt % V_STAGES) * L::OPERAND_BYTES;
#pragma unroll
                for (int s = 0; s < TILE / 16; ++s)   // 16 keys: 8 columns of P (two bfloat16 each), 16 rows of V of 128 bytes
                    umma_ts(tmem_o + g * HD, tmem_base + g * TILE + s * 8, desc_mn_major(vb + s * 16 * 128, ROWS * 128), idesc_pv, (!first || s > 0) ? 1u : 0u);
                umma_commit(bar_o + g);
            };
            bool ok = true;
            int base = 0, count[2] = {0, 0}, items_of[2] = {0, 0};   // tiles and items each query tile has worked on so far
            for (int j = 0; ok; ++j) {
                ok = mbar_wait(bar_item + (j & 1), (uint32_t)(j >> 1) & 1, abort_flag);
                if (!ok) break;
                const Item it = item_ring[j & 1];
                const int n_tiles = it.n_tiles, ta = it.tiles_a, tb = it.tiles_b;
                if (n_tiles < 0) break;
                // the item's Q tiles are in shared memory (the scores' columns are free: every P.V of the item before
                // has been issued, and the tensor core runs in order) and its first K tile has landed
                ok = mbar_wait(bar_q, (uint32_t)j & 1, abort_flag) && mbar_wait(bar_k + base % K_STAGES, (uint32_t)(base / K_STAGES) & 1, abort_flag);
                if (!ok) break;
                fence_after_sync();
                issue_qk(0, base);
                if (tb > 0) issue_qk(1, base);
                umma_commit(bar_kfree + base % K_STAGES);   // every product that reads the item's first K tile has been issued
                // an accumulator still holds the query tile's last item until its group has read it out
                if (ok && items_of[0] > 0) ok = mbar_wait(bar_epi + 0, (uint32_t)(items_of[0] - 1) & 1, abort_flag);
                if (ok && tb > 0 && items_of[1] > 0) ok = mbar_wait(bar_epi + 1, (uint32_t)(items_of[1] - 1) & 1, abort_flag);
                for (int t = 0; t < n_tiles && ok; ++t) {
                    const int gt = base + t;
                    const bool more = t + 1 < n_tiles;
                    if (more) {
                        ok = mbar_wait(bar_k + (gt + 1) % K_STAGES, (uint32_t)((gt + 1) / K_STAGES) & 1, abort_flag);
                        if (!ok) break;
                    }
                    ok = mbar_wait(bar_v + gt % V_STAGES, (uint32_t)(gt / V_STAGES) & 1, abort_flag);
                    if (!ok) break;
                    if (t < ta) {
                        ok = mbar_wait(bar_p + 0, (uint32_t)count[0] & 1, abort_flag);
                        if (!ok) break;
                        fence_after_sync();
                        issue_pv(0, gt, t == 0);
                        ++count[0];
                        if (t + 1 < ta) issue_qk(0, gt + 1);   // S_A is free: P_A(t) lies in it and the product above reads it first
                    }
                    if (t < tb) {
                        ok = mbar_wait(bar_p + 1, (uint32_t)count[1] & 1, abort_flag);
                        if (!ok) break;
                        fence_after_sync();
                        issue_pv(1, gt, t == 0);
                        ++count[1];
                        if (t + 1 < tb) issue_qk(1, gt + 1);
                    }
                    umma_commit(bar_vfree + gt % V_STAGES);          // every product that reads V(t) has been issued
                    if (more) umma_commit(bar_kfree + (gt + 1) % K_STAGES);   // and every one that reads K(t + 1)
                }
                base += n_tiles;
                items_of[0] += 1;                 // tile A has tiles in every item
                items_of[1] += tb > 0 ? 1 : 0;
            }
        }
    } else {
        // ---------------------------------------------------------------- TMA of K (warp 9) and V (warp 10) tiles
        // One box per page and 64-column half; the lanes of the warp issue the boxes of a tile side
        // by side (a single thread issuing them one after the other is the slower way: small boxes
        // are bound by issue latency, not by bandwidth).  The warps run ahead into the next item's tiles
        // as far as the stages allow, so an item's first keys are there when its Q tiles are.
        const int kv = warp - 9;
        const int stages = kv == 0 ? K_STAGES : V_STAGES;
        const int pages_per_tile = TILE / p.page_size;
        const int boxes = pages_per_tile * (HD / 64);
        const uint32_t box_bytes = (uint32_t)p.page_size * 128;              // page_size rows of 64 elements
        const int my_page = lane / (HD / 64), my_half = lane % (HD / 64);   // this lane's box of a tile
        bool ok = true;
        int base = 0;
        for (int j = 0; ok; ++j) {
            ok = mbar_wait(bar_item + (j & 1), (uint32_t)(j >> 1) & 1, abort_flag);
            if (!ok) break;
            const Item it = item_ring[j & 1];
            if (it.n_tiles < 0) break;
            const int* bt = p.block_table + (size_t)it.seq * p.table_width;
            for (int t = 0; t < it.n_tiles; ++t) {
                const int gt = base + t, st = gt % stages;
                uint64_t* bar = (kv == 0 ? bar_k : bar_v) + st;
                // this lane's page of the tile, looked up before the wait for the stage (which hides the lookup);
                // pages that hold keys no row of the block can see, or that the table does not name, are skipped
                const int lp = (it.tile_first + t) * pages_per_tile + my_page;
                const bool in_range = lane < boxes && lp * p.page_size <= it.block_last_pos && (lp + 1) * p.page_size > it.block_lo;
                const int page = (in_range && lp < p.table_width) ? bt[lp] : -1;
                const bool valid = in_range && page >= 0 && page < p.num_pages;
                if (in_range && !valid && kv == 0) report_status(p.status, SPY_STATUS_BAD_PAGE, it.tok0);
                const int count = __popc(__ballot_sync(0xffffffffu, valid));
                if (lane == 0) {
                    // K's stage is free when every Q.K of the tile `stages` back is complete, V's when every P.V is
                    if (gt >= stages) ok = mbar_wait((kv == 0 ? bar_kfree : bar_vfree) + st, (uint32_t)(gt / stages - 1) & 1, abort_flag);
                    if (ok) mbar_expect_tx(bar, (uint32_t)count * box_bytes);
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                if (valid) {
                    const int y = ((page * 2 + kv) * p.nkv + it.kvh) * p.page_size;
                    tma_load_2d((kv == 0 ? k_s : v_s) + st * L::OPERAND_BYTES + my_half * (ROWS * 128) + my_page * p.page_size * 128, &page_map, my_half * 64, y, bar);
                }
            }
            base += it.n_tiles;
        }
    }

    fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) {
            const unsigned long long t0 = global_timer();
            while (global_timer() - t0 < 2000000ull) { }   // let copies in flight land before the shared memory is released
            report_status(p.status, SPY_STATUS_WAIT_TIMEOUT, (int)blockIdx.x);
        }
        __syncthreads();
    }
    if (warp == 8) {
        fence_after_sync();
        tmem_dealloc(tmem_base, L::TMEM_COLS);
    }
}

}  // namespace


// Attention of a batch over its pages: prompt portions, any mix, single tokens included.
extern "C" int spy_attention_tc(const void* q, long long q_row_stride, void* out, const void* pages, const int* block_table, int table_width,
                                int page_size, int num_pages, int nh, int nkv, int hd, const int* positions, const int* q_start, int tokens,
                                int seqs, int window, float scale, int* status, cudaStream_t stream)
{
    if (tokens <= 0 || seqs <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) SPY_FAIL("attention_tc: %d query heads do not group over %d key/value heads", nh, nkv);
    const int G = nh / nkv;
    if (G > 16) SPY_FAIL("attention_tc: %d query heads per key/value head exceed 16", G);
    if (hd < 8 || hd > 128 || hd % 8 != 0) SPY_FAIL("attention_tc: head_dim %d is not a multiple of 8 between 8 and 128", hd);
    if (q_row_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(pages) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 15))
        SPY_FAIL("attention_tc: queries, pages and output must be 16-byte aligned with rows a multiple of 8 elements");
    if (page_size <= 0 || num_pages <= 0 || table_width <= 0) SPY_FAIL("attention_tc: page_size, num_pages and table_width must be positive");
    if (window < 0) SPY_FAIL("attention_tc: window %d must be 0 (none) or positive", window);
    const int Gp = G;   // rows a token takes in a query tile: one per head of the group (128 / G tokens a tile, the remainder of the rows stays empty)
    Params p;
    p.q = (const bf16*)q; p.q_stride = q_row_stride; p.out = (bf16*)out; p.block_table = block_table;
    p.positions = positions; p.q_start = q_start; p.status = status; p.table_width = table_width; p.page_size = page_size;
    p.num_pages = num_pages; p.nh = nh; p.nkv = nkv; p.G = G; p.Gp = Gp; p.S = seqs; p.window = window; p.hd = hd; p.scale_log2 = scale * LOG2E;
    if (page_size < 8 || page_size > TILE || TILE % page_size != 0)
        SPY_FAIL("attention_tc: page_size %d must be 8, 16, 32, 64 or 128 (one TMA box per page)", page_size);
    // the pages of this cache as one matrix [num_pages * 2 * nkv * page_size rows, hd]; a box is one page's rows x 64 columns
    // (columns beyond hd are outside the matrix and arrive as zeros: a head size below the tile's 64 or 128 is padded on the way in)
    tc::EncodeTiledFn encode = tc::encode_tiled_fn();
    if (encode == nullptr) SPY_FAIL("attention_tc: cuTensorMapEncodeTiled is not available from the driver");
    CUtensorMap page_map;
    {
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)num_pages * 2 * nkv * page_size};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)page_size};
        cuuint32_t elem[2] = {1, 1};
        CUresult r = encode(&page_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) SPY_FAIL("attention_tc: cuTensorMapEncodeTiled failed with code %d", (int)r);
    }
    SPY_ONCE_PER_DEVICE {
        SPY_CUDA(cudaFuncSetAttribute(attention_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<64>::TOTAL));
        SPY_CUDA(cudaFuncSetAttribute(attention_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<128>::TOTAL));
    }
    const int tokens_per_block = 2 * (BLOCK_ROWS / 2 / Gp);
    const long long blocks = (tokens + tokens_per_block - 1) / tokens_per_block + seqs;   // an upper bound without a host copy of q_start
    const long long items = blocks * nkv;
    if (items > 0x7fffffffLL) SPY_FAIL("attention_tc: the batch's %lld work items exceed the kernel's range", items);
    p.x_blocks = (int)blocks;
    p.items = (int)items;
    // one resident block per SM walks through the items (set-up once, the next item's keys requested while the
    // last tiles of the one before are worked on)
    const int sms = spy_sm_count();
    dim3 grid((unsigned)(items < sms ? items : sms));
    if (hd <= 64) spy_launch(attention_tc_kernel<64>, grid, dim3(NUM_THREADS), (size_t)Smem<64>::TOTAL, stream, page_map, p);
    else spy_launch(attention_tc_kernel<128>, grid, dim3(NUM_THREADS), (size_t)Smem<128>::TOTAL, stream, page_map, p);
    SPY_CHECK_LAUNCH("attention_tc");
    return 0;
}
