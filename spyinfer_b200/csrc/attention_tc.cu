// bfloat16 attention for prompt portions on the 5th-generation tensor cores (tcgen05), keys
// and values read from the paged cache.
//
// One block owns 128 rows = (128 / Gp) consecutive tokens of one sequence x the G query
// heads of one key/value head (Gp = G rounded up to a power of two), and walks the keys in
// tiles of 128:
//   S = Q . K^T      one 128 x 128 x head_dim product into tensor memory (tcgen05.mma, operands in
//                    shared memory, both K-major, 128-byte swizzle)
//   softmax          eight warps, TWO THREADS PER ROW, each with 64 of the row's 128 scores
//                    (tcgen05.ld): the halves exchange their maxima through shared memory, the
//                    running maximum and sum need no shuffles; exp2 on pre-scaled scores in 32-bit
//                    (packed f32x2 FMA/ADD and the 3-input max of sm_100 keep the instruction count
//                    down); the probabilities go BACK INTO TENSOR MEMORY as bfloat16 (tcgen05.st),
//                    over the scores they were made from
//   O += P . V       one 128 x head_dim x 128 product with P read from tensor memory; V's tile is
//                    used as it lies in the pages (head_dim contiguous: an MN-major operand), O
//                    stays in tensor memory
// P takes no shared memory, which leaves room for three stages of K and of V tiles: a tile is
// requested two to three tiles before the tensor core needs it, which is what hides the latency
// of its many small TMA boxes.
// The output is rescaled only when a row's maximum grew by more than 2^8 (the stale maximum
// keeps every probability below 256, harmless in bfloat16 and float32); then the row's two
// threads read, scale and write back their halves of O's row (tcgen05.ld / tcgen05.st).
// Scores and probabilities are double-buffered, so that the tensor
// cores compute Q.K of the next tile and P.V of the last one while the softmax warps work on
// the current one.  A ninth warp allocates tensor memory and issues the MMAs; two more bring
// the key and the value tiles in with TMA, one box of 64 columns x page_size rows per page and
// half of head_dim, straight from the paged cache (no cluster multicast), as soon as a stage
// is free.  Pages the block table does not name are skipped; the stages are zeroed once, so
// such rows hold finite values that the masks then exclude.
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

constexpr int ROWS = 128;            // query rows per block = UMMA M
constexpr int TILE = 128;            // keys per tile = UMMA N of the first product
constexpr int STAGES = 3;            // K and V tiles in flight
constexpr int SOFTMAX_THREADS = 256; // warps 0..7: Q load, softmax (two threads per row), epilogue
constexpr int NUM_THREADS = 352;     // warp 8: TMEM + MMA; warps 9, 10: TMA of K and of V
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;

struct Params {
    const bf16* q;
    long long q_stride;
    bf16* out;                 // [T, nh * HD]
    const int* block_table;    // [S, table_width]
    const int* positions;      // [T]
    const int* q_start;        // [S + 1]
    int* status;
    int table_width, page_size, num_pages, nh, nkv, G, Gp, S, window;
    int x_blocks, items;       // 128-row blocks along the tokens (an upper bound), and x_blocks * nkv work items
    float scale_log2;
};

// One work item: 128 query rows of one sequence and key/value head, and the key tiles they see.
struct Item {
    int seq, tok0, kvh, n_tiles, tile_first, block_lo, block_last_pos, tok_end;
};


// Byte offset of 16-byte chunk `chunk` (0 .. HD / 8 - 1, or 0 .. 15 for the 128-key P tile) of
// row `row` in a [128 rows][64-element halves] tile with 128-byte swizzle.
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk)
{
    return (uint32_t)((chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int HD> struct Smem {
    static constexpr int OPERAND_BYTES = ROWS * HD * 2;       // Q, K or V tile
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = Q_OFF + OPERAND_BYTES;            // STAGES stages
    static constexpr int V_OFF = K_OFF + STAGES * OPERAND_BYTES;   // STAGES stages
    // what the two threads of a row tell each other: bfloat16[2 score stages][2 halves][128 rows] maxima, at the end float[2 halves][128 rows] sums
    static constexpr int X_OFF = V_OFF + STAGES * OPERAND_BYTES;
    static constexpr int BAR_OFF = X_OFF + 2 * ROWS * 4;
    // barriers and the two work items (320 bytes), then slack to align the base to 1024 (the base is aligned to 128)
    static constexpr int TOTAL = BAR_OFF + 320 + 896;
    static constexpr int TMEM_COLS = 512;                     // S0, S1: 128 columns each (P_t over the first 64 of S_t); O: HD columns from 256
};

// Pipeline (tile t uses stage t & 1 of S and P, stage t % 3 of K and V):
//   softmax warps, iteration t:  wait S_t | read S_t, max, exchange, exp (registers) |
//                                if O must be rescaled: wait P.V_{t-1}, rescale | write P_t | signal
//   MMA thread:                  Q.K_0, Q.K_1, then for every t:  wait P_t and V_t | P.V_t | wait K_{t+2} | Q.K_{t+2}
// so the tensor cores work on P.V_{t-1} and Q.K_{t+1} while the softmax warps work on tile t.
template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, 1) attention_tc_kernel(const __grid_constant__ CUtensorMap page_map, const Params p)
{
    using L = Smem<HD>;
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __nv_bfloat16* xch = reinterpret_cast<__nv_bfloat16*>(smem + L::X_OFF);   // [2][2][ROWS]
    float* xsum = reinterpret_cast<float*>(smem + L::X_OFF);                  // [2][ROWS], after the last tile
    uint64_t* bar_k = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);   // [STAGES] K tile landed (TMA bytes)
    uint64_t* bar_v = bar_k + STAGES;                                   // [STAGES] V tile landed (TMA bytes)
    uint64_t* bar_kfree = bar_v + STAGES;                               // [STAGES] Q.K of the stage's tile complete (MMA commit)
    uint64_t* bar_vfree = bar_kfree + STAGES;                           // [STAGES] P.V of the stage's tile complete (MMA commit)
    uint64_t* bar_s = bar_vfree + STAGES;                               // [2] scores complete (MMA commit)
    uint64_t* bar_p = bar_s + 2;                                        // [2] probabilities written (256 arrivals)
    uint64_t* bar_o = bar_p + 2;                                        // [2] P.V complete (MMA commit)
    uint64_t* bar_x = bar_o + 2;                                        // [2] the halves' maxima are written (256 arrivals)
    uint64_t* bar_q = bar_x + 2;                                        // the item's Q tile is written (256 arrivals)
    uint64_t* bar_sum = bar_q + 1;                                      // the halves' sums of the item are written (256 arrivals)
    uint64_t* bar_item = bar_sum + 1;                                   // [2] the block's next work item is described (thread 0)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_item + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    Item* item_ring = reinterpret_cast<Item*>(tmem_slot + 2);           // [2]

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int tokens_per_block = ROWS / p.Gp;
    if (tid == 0) {
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(bar_k + i, 1);
            mbar_init(bar_v + i, 1);
            mbar_init(bar_kfree + i, 1);
            mbar_init(bar_vfree + i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_s + i, 1);
            mbar_init(bar_p + i, SOFTMAX_THREADS);
            mbar_init(bar_o + i, 1);
            mbar_init(bar_x + i, SOFTMAX_THREADS);
            mbar_init(bar_item + i, 1);
        }
        mbar_init(bar_q, SOFTMAX_THREADS);
        mbar_init(bar_sum, SOFTMAX_THREADS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) tmem_alloc(tmem_slot, L::TMEM_COLS);
    // rows of pages the block table does not name are never copied: keep them finite
    for (int i = tid; i < 2 * STAGES * L::OPERAND_BYTES / 16; i += NUM_THREADS) reinterpret_cast<uint4*>(smem + L::K_OFF)[i] = make_uint4(0, 0, 0, 0);
    fence_async_proxy();
    pdl_wait();   // everything below reads what earlier kernels wrote

    // The block's work items.  The items are numbered with the long ones first (in a causal prompt the
    // late rows see the most keys): item i is the block of rows x_blocks - 1 - i / nkv, counted through
    // the sequences, of key/value head i % nkv.  The block takes one item a round, forwards in even rounds
    // and backwards in odd ones, so that a long item of one round meets a short one of the next.
    const int G_blocks = (int)gridDim.x, blk = (int)blockIdx.x;
    auto item_index = [&](int k) { return k * G_blocks + ((k & 1) ? G_blocks - 1 - blk : blk); };
    // Thread 0 describes the block's (j + 1)-th item WITH TILES while the block works on the j-th; every role
    // waits for the description.  Rounds whose item has no tiles (x_blocks is an upper bound; a window may
    // leave a block without keys) are passed over here, so that every entry of the ring is real work: thread 0
    // can then never be two entries ahead of a role that has not read its entry yet.  After the last item an
    // entry with n_tiles = -1 ends the roles.
    int next_round = 0;   // thread 0 only
    auto describe_next = [&](int j) {
        Item it;
        it.seq = -1; it.tok0 = 0; it.kvh = 0; it.n_tiles = -1; it.tile_first = 0; it.block_lo = 0; it.block_last_pos = -1; it.tok_end = 0;
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
            it.block_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
            if (it.block_lo <= it.block_last_pos) {
                it.tile_first = it.block_lo / TILE;
                it.n_tiles = it.block_last_pos / TILE - it.tile_first + 1;
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
    // Every role walks the same entries j = 0, 1, ... and counts the same tiles: `base` tiles before the
    // current item's; the barriers' stages and phases follow the running tile number base + t.

    if (warp < 8) {
        // ---------------------------------------------------------------- loads, softmax, epilogue
        const int row = tid & (ROWS - 1), half = tid >> 7;    // this thread's query row = TMEM lane, and its half of the row's columns
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        constexpr int COLS = TILE / 2;       // scores per thread
        constexpr int OCOLS = HD / 2;        // output columns per thread
        bool alive = true, q_requested = false;
        int base = 0;
        // The item's Q tile: consecutive threads copy consecutive 16-byte pieces of a row.  It is requested as soon
        // as the item before has its last scores (every Q.K of that item is then complete), and so arrives
        // while that item's output is read and stored.
        auto request_q = [&](const Item& it) {
            constexpr int CPR = HD / 8;
            for (int idx = tid; idx < ROWS * CPR; idx += SOFTMAX_THREADS) {
                const int r = idx / CPR, c = idx % CPR;
                const int r_tok = it.tok0 + r / p.Gp, r_hg = r % p.Gp;
                const bool ok = r_tok < it.tok_end && r_hg < p.G;
                const bf16* src = p.q + (size_t)(ok ? r_tok : 0) * p.q_stride + (size_t)(it.kvh * p.G + (ok ? r_hg : 0)) * HD + c * 8;
                cp_async16(smem + L::Q_OFF + tile_offset(r, c), src, ok);
            }
        };
        for (int j = 0; alive; ++j) {
            alive = mbar_wait(bar_item + (j & 1), (uint32_t)(j >> 1) & 1, abort_flag);
            if (!alive) break;
            const Item it = item_ring[j & 1];
            if (it.n_tiles < 0) break;
            const int n_tiles = it.n_tiles, tile_first = it.tile_first, tok0 = it.tok0, tok_end = it.tok_end, kvh = it.kvh;
            const int tok = tok0 + row / p.Gp, hg = row % p.Gp;
            const bool row_ok = tok < tok_end && hg < p.G;
            const int head = kvh * p.G + hg;
            // the keys this row sees
            const int pos = row_ok ? min(p.positions[tok], it.block_last_pos) : -1;
            const int lo = max((row_ok && p.window > 0) ? max(0, p.positions[tok] - p.window + 1) : 0, it.block_lo);
            if (!q_requested) request_q(it);   // the block's first item
            asm volatile("cp.async.wait_all;" ::: "memory");
            fence_async_proxy();   // the MMA reads shared memory through the async proxy
            mbar_arrive(bar_q);
            if (tid == 0) describe_next(j + 1);   // while the first scores are on their way

            float m_used = -INFINITY, l = 0.f;   // the maximum the probabilities are taken against (equal in both threads of a row); this thread's share of their sum
            for (int t = 0; t < n_tiles; ++t) {
                const int gt = base + t, st = gt & 1;
                const uint32_t ph = (uint32_t)(gt >> 1) & 1;
                alive = mbar_wait(bar_s + st, ph, abort_flag);          // S_t is complete
                if (!alive) break;
                fence_after_sync();
                const int key0 = (tile_first + t) * TILE + half * COLS;
                // This thread's 64 raw scores (masked where the tile is not visible whole to every row of the warp).
                // The scale is folded into the exponent's argument, exp2(s * scale - m), one packed FMA for two
                // scores; the maximum is taken on the raw scores (the scale is positive) by 3-input max in four
                // independent chains; the sum runs in two packed accumulators.
                uint32_t sc[COLS];
#pragma unroll
                for (int c = 0; c < COLS; c += 32) tmem_load<32>(tmem_base + st * TILE + lane_addr + half * COLS + c, *reinterpret_cast<uint32_t(*)[32]>(&sc[c]));
                tmem_wait_ld();
                const bool whole = __all_sync(0xffffffffu, !row_ok || (key0 >= lo && key0 + COLS - 1 <= pos));
                if (!whole) {
#pragma unroll
                    for (int i = 0; i < COLS; ++i) {
                        const int j = key0 + i;
                        if (!(j <= pos && j >= lo)) sc[i] = 0xff800000u;   // -inf
                    }
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int i = 0; i < COLS; i += 8) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) mx4[c] = max3(mx4[c], __uint_as_float(sc[i + 2 * c]), __uint_as_float(sc[i + 2 * c + 1]));
                }
                // The halves tell each other their maxima rounded UP to bfloat16: any common upper bound serves
                // as the value the exponentials are taken against, and both threads must use the same one.
                const __nv_bfloat16 mine = __float2bfloat16_ru(fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])));
                xch[(st * 2 + half) * ROWS + row] = mine;
                mbar_arrive(bar_x + st);
                alive = mbar_wait(bar_x + st, ph, abort_flag);
                if (!alive) break;
                const float mx = fmaxf(__bfloat162float(mine), __bfloat162float(xch[(st * 2 + (half ^ 1)) * ROWS + row])) * p.scale_log2;
                // the maximum in use moves only when the row's maximum grew by more than the threshold (or from nothing)
                const float m_new = fmaxf(m_used, mx);
                const bool grow = m_new > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && m_new != -INFINITY);
                const float alpha = grow ? (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new)) : 1.f;
                if (grow) {
                    l *= alpha;
                    m_used = m_new;
                }
                const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
                const uint64_t scale2 = pack2(p.scale_log2, p.scale_log2), neg2 = pack2(neg_m, neg_m);
                uint64_t sum2[2] = {0ull, 0ull};
                uint32_t packed[COLS / 2];
#pragma unroll
                for (int i = 0; i < COLS; i += 2) {
                    float a0, a1;
                    unpack2(fma2(pack2(__uint_as_float(sc[i]), __uint_as_float(sc[i + 1])), scale2, neg2), a0, a1);
                    const float p0 = fast_exp2(a0), p1 = fast_exp2(a1);
                    sum2[(i >> 1) & 1] = add2(sum2[(i >> 1) & 1], pack2(p0, p1));
                    packed[i / 2] = pack_bf16(p0, p1);
                }
                {
                    float s0, s1;
                    unpack2(add2(sum2[0], sum2[1]), s0, s1);
                    l += s0 + s1;
                }
                // Only a rescale of O has to wait for P.V of tile t-1, so in the common case P_t is ready before
                // that product ends and the next one follows it without a gap.
                if (t > 0 && __any_sync(0xffffffffu, grow)) {   // the warp with the row's other half decides the same
                    alive = mbar_wait(bar_o + ((gt - 1) & 1), (uint32_t)((gt - 1) >> 1) & 1, abort_flag);
                    if (!alive) break;
                    fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < OCOLS; c += 32) {
                        uint32_t r[32];
                        tmem_load<32>(tmem_o + lane_addr + half * OCOLS + c, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_store<32>(tmem_o + lane_addr + half * OCOLS + c, r);
                        tmem_wait_st();
                    }
                }
                // P_t over the first 64 columns of S_t: both threads of the row have their scores in registers
                // (the partner loaded its own before it arrived at the exchange)
#pragma unroll
                for (int c = 0; c < COLS / 2; c += 32)
                    tmem_store<32>(tmem_base + st * TILE + lane_addr + half * (COLS / 2) + c, *reinterpret_cast<uint32_t(*)[32]>(&packed[c]));
                tmem_wait_st();
                fence_before_sync();
                mbar_arrive(bar_p + st);
            }
            if (!alive) break;
            // ---- the next item's Q tile is requested ...
            alive = mbar_wait(bar_item + ((j + 1) & 1), (uint32_t)((j + 1) >> 1) & 1, abort_flag);
            if (!alive) break;
            q_requested = item_ring[(j + 1) & 1].n_tiles > 0;
            if (q_requested) request_q(item_ring[(j + 1) & 1]);
            // ---- ... and this item's epilogue runs meanwhile: O / l
            const int gl = base + n_tiles - 1;
            alive = mbar_wait(bar_o + (gl & 1), (uint32_t)(gl >> 1) & 1, abort_flag);
            if (!alive) break;
            fence_after_sync();
            xsum[half * ROWS + row] = l;   // every thread has read the maxima of the last tile: it wrote P after that, and P.V is complete
            mbar_arrive(bar_sum);
            alive = mbar_wait(bar_sum, (uint32_t)j & 1, abort_flag);
            if (!alive) break;
            {
                const float sum = half == 0 ? l + xsum[ROWS + row] : xsum[row] + l;   // the same order in both threads
                const float inv = sum > 0.f ? 1.f / sum : 0.f;
                bf16* dst = p.out + ((size_t)(row_ok ? tok : 0) * p.nh + head) * HD + half * OCOLS;
#pragma unroll 1
                for (int c = 0; c < OCOLS; c += 32) {
                    uint32_t r[32];
                    tmem_load<32>(tmem_o + lane_addr + half * OCOLS + c, r);
                    tmem_wait_ld();
                    if (!row_ok) continue;
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) {
                        uint4 v;
                        v.x = pack_bf16(__uint_as_float(r[8 * q4]) * inv, __uint_as_float(r[8 * q4 + 1]) * inv);
                        v.y = pack_bf16(__uint_as_float(r[8 * q4 + 2]) * inv, __uint_as_float(r[8 * q4 + 3]) * inv);
                        v.z = pack_bf16(__uint_as_float(r[8 * q4 + 4]) * inv, __uint_as_float(r[8 * q4 + 5]) * inv);
                        v.w = pack_bf16(__uint_as_float(r[8 * q4 + 6]) * inv, __uint_as_float(r[8 * q4 + 7]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + 8 * q4) = v;
                    }
                }
            }
            // the next item's first P.V overwrites O: it needs that item's probabilities, which every thread writes
            // only after it has read its part of O here
            fence_before_sync();
            base += n_tiles;
        }
    } else if (warp == 8) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc_qk = instr_desc_bf16(ROWS, TILE, false, false), idesc_pv = instr_desc_bf16(ROWS, HD, false, true);
            auto issue_qk = [&](int gt) {   // gt: the running tile number
                const uint32_t kb = k_s + (gt % STAGES) * L::OPERAND_BYTES;
#pragma unroll
                for (int s = 0; s < HD / 16; ++s) {
                    const uint32_t off = (s >> 2) * (ROWS * 128) + (s & 3) * 32;   // 64-element half, then 32 bytes per 16 elements
                    umma(tmem_base + (gt & 1) * TILE, desc_k_major(q_s + off), desc_k_major(kb + off), idesc_qk, s > 0 ? 1u : 0u);
                }
                umma_commit(bar_s + (gt & 1));
                umma_commit(bar_kfree + gt % STAGES);
            };
            bool ok = true;
            int base = 0;
            for (int j = 0; ok; ++j) {
                ok = mbar_wait(bar_item + (j & 1), (uint32_t)(j >> 1) & 1, abort_flag);
                if (!ok) break;
                const int n_tiles = item_ring[j & 1].n_tiles;
                if (n_tiles < 0) break;
                // the item's Q tile is in shared memory (and the scores' stages are free: every P.V of the item before
                // has been issued, and the tensor core runs in order)
                ok = mbar_wait(bar_q, (uint32_t)j & 1, abort_flag) && mbar_wait(bar_k + base % STAGES, (uint32_t)(base / STAGES) & 1, abort_flag);
                if (ok) {
                    fence_after_sync();
                    issue_qk(base);
                }
                if (ok && n_tiles > 1) {
                    ok = mbar_wait(bar_k + (base + 1) % STAGES, (uint32_t)((base + 1) / STAGES) & 1, abort_flag);
                    if (ok) {
                        fence_after_sync();
                        issue_qk(base + 1);
                    }
                }
                for (int t = 0; t < n_tiles && ok; ++t) {
                    const int gt = base + t, st = gt & 1, stage = gt % STAGES;
                    ok = mbar_wait(bar_p + st, (uint32_t)(gt >> 1) & 1, abort_flag);
                    ok = ok && mbar_wait(bar_v + stage, (uint32_t)(gt / STAGES) & 1, abort_flag);
                    if (!ok) break;
                    fence_after_sync();
                    const uint32_t vb = v_s + stage * L::OPERAND_BYTES;
#pragma unroll
                    for (int s = 0; s < TILE / 16; ++s)   // 16 keys: 8 columns of P (two bfloat16 each), 16 rows of V of 128 bytes
                        umma_ts(tmem_o, tmem_base + st * TILE + s * 8, desc_mn_major(vb + s * 16 * 128, ROWS * 128), idesc_pv, (t > 0 || s > 0) ? 1u : 0u);
                    umma_commit(bar_o + st);
                    umma_commit(bar_vfree + stage);
                    if (t + 2 < n_tiles) {
                        // S's stage st is free: P_t lies in it and the product above reads it first (the tensor core runs in order)
                        ok = mbar_wait(bar_k + (gt + 2) % STAGES, (uint32_t)((gt + 2) / STAGES) & 1, abort_flag);
                        if (!ok) break;
                        fence_after_sync();
                        issue_qk(gt + 2);
                    }
                }
                base += n_tiles;
            }
        }
    } else {
        // ---------------------------------------------------------------- TMA of K (warp 9) and V (warp 10) tiles
        // One box per page and 64-column half; the lanes of the warp issue the boxes of a tile side
        // by side (a single thread issuing them one after the other is the slower way: small boxes
        // are bound by issue latency, not by bandwidth).  The warps run ahead into the next item's tiles
        // as far as the stages allow, so an item's first keys are there when its Q tile is.
        const int kv = warp - 9;
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
                const int gt = base + t, st = gt % STAGES;
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
                    // K's stage is free when Q.K of the tile three back is complete, V's when its P.V is
                    if (gt >= STAGES) ok = mbar_wait((kv == 0 ? bar_kfree : bar_vfree) + st, (uint32_t)(gt / STAGES - 1) & 1, abort_flag);
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
    if (hd != 64 && hd != 128) SPY_FAIL("attention_tc: head_dim %d is not 64 or 128", hd);
    if (q_row_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(pages) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 15))
        SPY_FAIL("attention_tc: queries, pages and output must be 16-byte aligned with rows a multiple of 8 elements");
    if (page_size <= 0 || num_pages <= 0 || table_width <= 0) SPY_FAIL("attention_tc: page_size, num_pages and table_width must be positive");
    if (window < 0) SPY_FAIL("attention_tc: window %d must be 0 (none) or positive", window);
    int Gp = 1;
    while (Gp < G) Gp *= 2;
    Params p;
    p.q = (const bf16*)q; p.q_stride = q_row_stride; p.out = (bf16*)out; p.block_table = block_table;
    p.positions = positions; p.q_start = q_start; p.status = status; p.table_width = table_width; p.page_size = page_size;
    p.num_pages = num_pages; p.nh = nh; p.nkv = nkv; p.G = G; p.Gp = Gp; p.S = seqs; p.window = window; p.scale_log2 = scale * LOG2E;
    if (page_size < 8 || page_size > TILE || TILE % page_size != 0)
        SPY_FAIL("attention_tc: page_size %d must be 8, 16, 32, 64 or 128 (one TMA box per page)", page_size);
    // the pages of this cache as one matrix [num_pages * 2 * nkv * page_size rows, hd]; a box is one page's rows x 64 columns
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
    const int tokens_per_block = ROWS / Gp;
    const long long blocks = (tokens + tokens_per_block - 1) / tokens_per_block + seqs;   // an upper bound without a host copy of q_start
    const long long items = blocks * nkv;
    if (items > 0x7fffffffLL) SPY_FAIL("attention_tc: the batch's %lld work items exceed the kernel's range", items);
    p.x_blocks = (int)blocks;
    p.items = (int)items;
    // one resident block per SM walks through the items (set-up once, the next item's keys requested while the
    // last tiles of the one before are worked on)
    const int sms = spy_sm_count();
    dim3 grid((unsigned)(items < sms ? items : sms));
    if (hd == 64) spy_launch(attention_tc_kernel<64>, grid, dim3(NUM_THREADS), (size_t)Smem<64>::TOTAL, stream, page_map, p);
    else spy_launch(attention_tc_kernel<128>, grid, dim3(NUM_THREADS), (size_t)Smem<128>::TOTAL, stream, page_map, p);
    SPY_CHECK_LAUNCH("attention_tc");
    return 0;
}
