// bfloat16 attention for prompt portions on the 5th-generation tensor cores (tcgen05), keys
// and values read from the paged cache.
//
// One block owns 128 rows = (128 / Gp) consecutive tokens of one sequence x the G query
// heads of one key/value head (Gp = G rounded up to a power of two), and walks the keys in
// tiles of 128:
//   S = Q . K^T      one 128 x 128 x head_dim product into tensor memory (tcgen05.mma, operands in
//                    shared memory, both K-major, 128-byte swizzle)
//   softmax          four warps, ONE ROW PER THREAD: tcgen05.ld brings the row's 128 scores, so the
//                    running maximum and sum need no shuffles; exp2 on pre-scaled scores in 32-bit;
//                    the probabilities go to shared memory as bfloat16
//   O += P . V       one 128 x head_dim x 128 product; V's tile is used as it lies in the pages
//                    (head_dim contiguous: an MN-major operand), O stays in tensor memory
// The output is rescaled only when a row's maximum grew by more than 2^8 (the stale maximum
// keeps every probability below 256, harmless in bfloat16 and float32); then the warp reads,
// scales and writes back its rows of O (tcgen05.ld / tcgen05.st).
// Scores, probabilities and the key and value tiles are double-buffered, so that the tensor
// cores compute Q.K of the next tile and P.V of the last one while the softmax warps work on
// the current one.  A fifth warp allocates tensor memory and issues the MMAs; two more bring
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

SPY_MODULE(spy_attention_tc)

namespace {

constexpr int ROWS = 128;          // query rows per block = UMMA M
constexpr int TILE = 128;          // keys per tile = UMMA N of the first product
constexpr int NUM_THREADS = 224;   // warps 0..3: Q load, softmax, epilogue; warp 4: TMEM + MMA; warps 5, 6: TMA of K and of V
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

struct Params {
    const bf16* q;
    long long q_stride;
    bf16* out;                 // [T, nh * HD]
    const bf16* pages;         // [num_pages][2][nkv][page_size][HD]
    const int* block_table;    // [S, table_width]
    const int* positions;      // [T]
    const int* q_start;        // [S + 1]
    int* status;
    float* part_o;             // split mode: [T][nh][max_splits][HD] unnormalised partial outputs
    float* part_ml;            //             [T][nh][max_splits][2]  (maximum in the log2 domain, sum)
    int table_width, page_size, num_pages, nh, nkv, G, Gp, S, window, split_keys, max_splits;
    float scale_log2;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long global_timer()
{
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag)
{
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer();
    uint32_t spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 0x3ff) == 0) {
            if (*abort_flag) return false;
            if (global_timer() - t0 > WAIT_LIMIT_NS) {
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, bool valid)
{
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(smem_dst)), "l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Shared-memory matrix descriptors (128-byte swizzle; 8 rows of 128 bytes form a 1024-byte group).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;                 // leading byte offset: unused for swizzled K-major
    d |= (uint64_t)(1024 >> 4) << 32;       // stride byte offset: next group of 8 rows
    d |= (uint64_t)1 << 46;                 // descriptor version of sm_100
    d |= (uint64_t)2 << 61;                 // SWIZZLE_128B
    return d;
}
// MN-major: the 128-byte rows run along the MN dimension (64 elements), 8 rows along K form a
// group; leading byte offset = next block of 64 MN elements, stride byte offset = next 8 K rows.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t addr, uint32_t lbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr & 0x3FFFF) >> 4);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__device__ __forceinline__ uint32_t instr_desc(int n, bool b_mn_major)
{
    uint32_t d = 0;
    d |= 1u << 4;                      // accumulator F32
    d |= 1u << 7;                      // A BF16
    d |= 1u << 10;                     // B BF16
    if (b_mn_major) d |= 1u << 16;     // B is MN-major
    d |= (uint32_t)(n >> 3) << 17;     // N
    d |= (uint32_t)(ROWS >> 4) << 24;  // M = 128
    return d;
}

__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_load_32(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_load_32_nowait(uint32_t taddr, uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}

__device__ __forceinline__ void tmem_store_32(uint32_t taddr, const uint32_t (&r)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]),
          "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]),
          "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}

// Byte offset of 16-byte chunk `chunk` (0 .. HD / 8 - 1, or 0 .. 15 for the 128-key P tile) of
// row `row` in a [128 rows][64-element halves] tile with 128-byte swizzle.
__device__ __forceinline__ uint32_t tile_offset(int row, int chunk)
{
    return (uint32_t)((chunk >> 3) * (ROWS * 128) + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
}

template <int HD> struct Smem {
    static constexpr int OPERAND_BYTES = ROWS * HD * 2;       // Q, K or V tile
    static constexpr int P_BYTES = ROWS * TILE * 2;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = Q_OFF + OPERAND_BYTES;       // two stages
    static constexpr int V_OFF = K_OFF + 2 * OPERAND_BYTES;   // two stages
    static constexpr int P_OFF = V_OFF + 2 * OPERAND_BYTES;   // two stages
    static constexpr int BAR_OFF = P_OFF + 2 * P_BYTES;
    static constexpr int TOTAL = BAR_OFF + 192 + 1024;        // barriers, then slack to align the base to 1024
    static constexpr int TMEM_COLS = 512;                     // S0, S1: 128 columns each; O: HD columns from 256
};

// Pipeline (tile t uses stage t & 1 of K, V, S and P):
//   softmax warps, iteration t:  wait S_t | request K_{t+2} | read S_t, max, exp (registers) |
//                                wait P.V_{t-1} | rescale O if needed | request V_{t+1} | write P_t | signal
//   MMA thread:                  Q.K_0, Q.K_1, then for every t:  wait P_t and V_t | P.V_t | wait K_{t+2} | Q.K_{t+2}
// so the tensor cores work on P.V_{t-1} and Q.K_{t+1} while the softmax warps work on tile t.
// SPLIT (decoding: every sequence brings one token): grid (sequence, kv head, split); the block
// takes the keys of split z only, its rows are the G heads of the one token (the first warp
// alone does the softmax), and when the token's keys span several splits the unnormalised
// output with its maximum and sum goes to scratch for attention_tc_merge_kernel.
template <int HD, bool SPLIT>
__global__ void __launch_bounds__(NUM_THREADS, 1) attention_tc_kernel(const __grid_constant__ CUtensorMap page_map, const Params p)
{
    using L = Smem<HD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bar_k = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);   // [2] K tile landed (TMA bytes)
    uint64_t* bar_v = bar_k + 2;                                        // [2] V tile landed (TMA bytes)
    uint64_t* bar_s = bar_v + 2;                                        // [2] scores complete (MMA commit)
    uint64_t* bar_p = bar_s + 2;                                        // [2] probabilities written (128 arrivals)
    uint64_t* bar_o = bar_p + 2;                                        // [2] P.V complete (MMA commit)
    uint64_t* bar_q = bar_o + 2;                                        // Q tile written (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_q + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* s_info = reinterpret_cast<int*>(tmem_slot + 2);                // seq, first token of the block

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int tokens_per_block = SPLIT ? 1 : ROWS / p.Gp;
    constexpr int SOFTMAX_WARPS = SPLIT ? 1 : 4;
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_k + i, 1);
            mbar_init(bar_v + i, 1);
            mbar_init(bar_s + i, 1);
            mbar_init(bar_p + i, SOFTMAX_WARPS * 32);
            mbar_init(bar_o + i, 1);
        }
        mbar_init(bar_q, ROWS);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)L::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    // rows of pages the block table does not name are never copied: keep them finite
    for (int i = tid; i < 4 * L::OPERAND_BYTES / 16; i += NUM_THREADS) reinterpret_cast<uint4*>(smem + L::K_OFF)[i] = make_uint4(0, 0, 0, 0);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    pdl_wait();   // everything below reads what earlier kernels wrote
    if (tid == 0) {
        int b = blockIdx.x, seq = -1, tok0 = 0;
        if constexpr (SPLIT) {
            seq = b;
            tok0 = p.q_start[b];
        } else {
            for (int s = 0; s < p.S; ++s) {
                const int n = p.q_start[s + 1] - p.q_start[s];
                const int blocks = (n + tokens_per_block - 1) / tokens_per_block;
                if (b < blocks) { seq = s; tok0 = p.q_start[s] + b * tokens_per_block; break; }
                b -= blocks;
            }
        }
        s_info[0] = seq;
        s_info[1] = tok0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 2 * TILE;
    const int seq = s_info[0], tok0 = s_info[1];
    const int kvh = blockIdx.y;

    int n_tiles = 0, tile_first = 0, block_lo = 0, block_last_pos = -1, tok_end = 0;
    int z_first = 0, z_last = 0;
    if (seq >= 0) {
        tok_end = SPLIT ? tok0 + 1 : p.q_start[seq + 1];
        const int first_pos = p.positions[tok0];
        block_last_pos = p.positions[min(tok_end, tok0 + tokens_per_block) - 1];
        block_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
        if constexpr (SPLIT) {
            z_first = block_lo / p.split_keys;
            z_last = block_last_pos / p.split_keys;
            const int z = blockIdx.z;
            block_lo = max(block_lo, z * p.split_keys);
            block_last_pos = min(block_last_pos, (z + 1) * p.split_keys - 1);
        }
        if (block_lo <= block_last_pos) {
            tile_first = block_lo / TILE;
            n_tiles = block_last_pos / TILE - tile_first + 1;
        }
    }
    const uint32_t q_s = smem_u32(smem + L::Q_OFF), k_s = smem_u32(smem + L::K_OFF), v_s = smem_u32(smem + L::V_OFF),
                   p_s = smem_u32(smem + L::P_OFF);

    if (warp < 4 && seq >= 0 && n_tiles > 0) {
        // ---------------------------------------------------------------- loads, softmax, epilogue
        const int row = tid;                                  // this thread's query row = TMEM lane
        const int tok = tok0 + row / p.Gp, hg = row % p.Gp;
        const bool row_ok = tok < tok_end && hg < p.G;
        const int head = kvh * p.G + hg;
        // the keys this row sees, within the block's range (a split's range when decoding)
        const int pos = row_ok ? min(p.positions[tok], block_last_pos) : -1;
        const int lo = max((row_ok && p.window > 0) ? max(0, p.positions[tok] - p.window + 1) : 0, block_lo);
        // the Q tile: consecutive threads copy consecutive 16-byte pieces of a row
        constexpr int CPR = HD / 8;
        for (int idx = tid; idx < ROWS * CPR; idx += ROWS) {
            const int r = idx / CPR, c = idx % CPR;
            const int r_tok = tok0 + r / p.Gp, r_hg = r % p.Gp;
            const bool ok = r_tok < tok_end && r_hg < p.G;
            const bf16* src = p.q + (size_t)(ok ? r_tok : 0) * p.q_stride + (size_t)(kvh * p.G + (ok ? r_hg : 0)) * HD + c * 8;
            cp_async16(smem + L::Q_OFF + tile_offset(r, c), src, ok);
        }
        asm volatile("cp.async.wait_all;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads shared memory through the async proxy
        mbar_arrive(bar_q);

        float m_used = -INFINITY, l = 0.f;   // the maximum the probabilities are taken against, and their sum
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        bool alive = true;
        for (int t = 0; t < n_tiles && warp < SOFTMAX_WARPS; ++t) {
            const int st = t & 1;
            const uint32_t ph = (uint32_t)(t >> 1) & 1;
            alive = mbar_wait(bar_s + st, ph, abort_flag);          // S_t is complete
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int key0 = (tile_first + t) * TILE;
            // the row's 128 scores, scaled (and masked where the tile is not visible whole to every row of the warp)
            float sc[TILE];
#pragma unroll
            for (int c = 0; c < TILE; c += 32) {
                uint32_t r[32];
                tmem_load_32_nowait(tmem_base + st * TILE + lane_addr + c, r);
#pragma unroll
                for (int i = 0; i < 32; ++i) sc[c + i] = __uint_as_float(r[i]);
            }
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            const bool whole = __all_sync(0xffffffffu, !row_ok || (key0 >= lo && key0 + TILE - 1 <= pos));
            float mx = -INFINITY;
            if (whole) {
#pragma unroll
                for (int i = 0; i < TILE; ++i) {
                    sc[i] *= p.scale_log2;
                    mx = fmaxf(mx, sc[i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < TILE; ++i) {
                    const int j = key0 + i;
                    sc[i] = (j <= pos && j >= lo) ? sc[i] * p.scale_log2 : -INFINITY;
                    mx = fmaxf(mx, sc[i]);
                }
            }
            // the maximum in use moves only when the row's maximum grew by more than the threshold (or from nothing)
            const float m_new = fmaxf(m_used, mx);
            const bool grow = m_new > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && m_new != -INFINITY);
            const float alpha = grow ? (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new)) : 1.f;
            if (grow) {
                l *= alpha;
                m_used = m_new;
            }
            const float m_sub = m_used == -INFINITY ? 0.f : m_used;
            uint32_t packed[TILE / 2];
#pragma unroll
            for (int i = 0; i < TILE; i += 2) {
                const float p0 = fast_exp2(sc[i] - m_sub), p1 = fast_exp2(sc[i + 1] - m_sub);
                l += p0 + p1;
                packed[i / 2] = pack_bf16(p0, p1);
            }
            // P.V of tile t-1 must be complete before O is rescaled and (two tiles back, implied)
            // before P's stage st is rewritten
            if (t > 0) {
                alive = mbar_wait(bar_o + ((t - 1) & 1), (uint32_t)((t - 1) >> 1) & 1, abort_flag);
                if (!alive) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            if (t > 0 && __any_sync(0xffffffffu, grow)) {
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    uint32_t r[32];
                    tmem_load_32(tmem_o + lane_addr + c, r);
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_store_32(tmem_o + lane_addr + c, r);
                }
            }
            uint8_t* pdst = smem + L::P_OFF + st * L::P_BYTES;
#pragma unroll
            for (int c8 = 0; c8 < TILE / 8; ++c8)
                *reinterpret_cast<uint4*>(pdst + tile_offset(row, c8)) =
                    make_uint4(packed[4 * c8], packed[4 * c8 + 1], packed[4 * c8 + 2], packed[4 * c8 + 3]);
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar_p + st);
        }
        // ---- epilogue: O / l, or the partial result of this split
        if (warp < SOFTMAX_WARPS) {
            if (alive) alive = mbar_wait(bar_o + ((n_tiles - 1) & 1), (uint32_t)((n_tiles - 1) >> 1) & 1, abort_flag);
            if (alive) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const bool direct = !SPLIT || z_first == z_last;
                const float inv = direct ? (l > 0.f ? 1.f / l : 0.f) : 1.f;
                bf16* dst = p.out + ((size_t)(row_ok ? tok : 0) * p.nh + head) * HD;
                const size_t slot = SPLIT ? ((size_t)(row_ok ? tok : 0) * p.nh + head) * p.max_splits + blockIdx.z : 0;
#pragma unroll 1
                for (int c = 0; c < HD; c += 32) {
                    uint32_t r[32];
                    tmem_load_32(tmem_o + lane_addr + c, r);
                    if (!row_ok) continue;
                    if (direct) {
#pragma unroll
                        for (int q4 = 0; q4 < 4; ++q4) {
                            uint4 v;
                            v.x = pack_bf16(__uint_as_float(r[8 * q4]) * inv, __uint_as_float(r[8 * q4 + 1]) * inv);
                            v.y = pack_bf16(__uint_as_float(r[8 * q4 + 2]) * inv, __uint_as_float(r[8 * q4 + 3]) * inv);
                            v.z = pack_bf16(__uint_as_float(r[8 * q4 + 4]) * inv, __uint_as_float(r[8 * q4 + 5]) * inv);
                            v.w = pack_bf16(__uint_as_float(r[8 * q4 + 6]) * inv, __uint_as_float(r[8 * q4 + 7]) * inv);
                            *reinterpret_cast<uint4*>(dst + c + 8 * q4) = v;
                        }
                    } else {
                        float4* po = reinterpret_cast<float4*>(p.part_o + slot * HD + c);
#pragma unroll
                        for (int q4 = 0; q4 < 8; ++q4)
                            po[q4] = make_float4(__uint_as_float(r[4 * q4]), __uint_as_float(r[4 * q4 + 1]), __uint_as_float(r[4 * q4 + 2]),
                                                 __uint_as_float(r[4 * q4 + 3]));
                    }
                }
                if (SPLIT && !direct && row_ok) {
                    p.part_ml[slot * 2] = m_used;
                    p.part_ml[slot * 2 + 1] = l;
                }
            }
        }
    } else if (warp == 4 && seq >= 0 && n_tiles > 0) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc_qk = instr_desc(TILE, false), idesc_pv = instr_desc(HD, true);
            auto issue_qk = [&](int t) {
                const uint32_t kb = k_s + (t & 1) * L::OPERAND_BYTES;
#pragma unroll
                for (int s = 0; s < HD / 16; ++s) {
                    const uint32_t off = (s >> 2) * (ROWS * 128) + (s & 3) * 32;   // 64-element half, then 32 bytes per 16 elements
                    umma(tmem_base + (t & 1) * TILE, desc_k_major(q_s + off), desc_k_major(kb + off), idesc_qk, s > 0 ? 1u : 0u);
                }
                umma_commit(bar_s + (t & 1));
            };
            bool ok = mbar_wait(bar_q, 0, abort_flag) && mbar_wait(bar_k + 0, 0, abort_flag);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_qk(0);
            }
            if (ok && n_tiles > 1) {
                ok = mbar_wait(bar_k + 1, 0, abort_flag);
                if (ok) {
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_qk(1);
                }
            }
            for (int t = 0; t < n_tiles && ok; ++t) {
                const int st = t & 1;
                const uint32_t ph = (uint32_t)(t >> 1) & 1;
                ok = mbar_wait(bar_p + st, ph, abort_flag) && mbar_wait(bar_v + st, ph, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t vb = v_s + st * L::OPERAND_BYTES, pb = p_s + st * L::P_BYTES;
#pragma unroll
                for (int s = 0; s < TILE / 16; ++s) {
                    const uint32_t a_off = (s >> 2) * (ROWS * 128) + (s & 3) * 32;   // P: 16 keys = 32 bytes along its rows
                    const uint32_t b_off = s * 16 * 128;                             // V: 16 key rows of 128 bytes
                    umma(tmem_o, desc_k_major(pb + a_off), desc_mn_major(vb + b_off, ROWS * 128), idesc_pv, (t > 0 || s > 0) ? 1u : 0u);
                }
                umma_commit(bar_o + st);
                if (t + 2 < n_tiles) {
                    ok = mbar_wait(bar_k + st, (uint32_t)((t + 2) >> 1) & 1, abort_flag);   // S's stage st is free: P_t was read from it
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_qk(t + 2);
                }
            }
        }
    }

    else if (warp >= 5 && seq >= 0 && n_tiles > 0) {
        // ---------------------------------------------------------------- TMA of K (warp 5) and V (warp 6) tiles
        // One box per page and 64-column half; the lanes of the warp issue the boxes of a tile side
        // by side (a single thread issuing them one after the other is the slower way: small boxes
        // are bound by issue latency, not by bandwidth).
        const int kv = warp - 5;
        const int* bt = p.block_table + (size_t)seq * p.table_width;
        const int pages_per_tile = TILE / p.page_size;
        const int boxes = pages_per_tile * (HD / 64);
        const uint32_t box_bytes = (uint32_t)p.page_size * 128;              // page_size rows of 64 elements
        bool ok = true;
        for (int t = 0; t < n_tiles; ++t) {
            const int st = t & 1;
            const int first_lp = (tile_first + t) * pages_per_tile;
            uint64_t* bar = (kv == 0 ? bar_k : bar_v) + st;
            if (lane == 0) {
                // K's stage is free when Q.K of tile t-2 is complete, V's when P.V of tile t-2 is
                if (t >= 2) ok = mbar_wait((kv == 0 ? bar_s : bar_o) + st, (uint32_t)((t - 2) >> 1) & 1, abort_flag);
                if (ok) {
                    int valid = 0;   // pages of this tile that the block table names and that hold keys some row can see
                    for (int i = 0; i < pages_per_tile; ++i) {
                        const int lp = first_lp + i;
                        const int page = lp < p.table_width ? bt[lp] : -1;
                        const bool in_range = lp * p.page_size <= block_last_pos && (lp + 1) * p.page_size > block_lo;
                        if (in_range && (page < 0 || page >= p.num_pages)) report_status(p.status, SPY_STATUS_BAD_PAGE, tok0);
                        if (in_range && page >= 0 && page < p.num_pages) ++valid;
                    }
                    mbar_expect_tx(bar, (uint32_t)valid * box_bytes * (HD / 64));
                }
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) break;
            const uint32_t stage = (kv == 0 ? k_s : v_s) + st * L::OPERAND_BYTES;
            for (int b = lane; b < boxes; b += 32) {
                const int i = b / (HD / 64), h = b % (HD / 64);
                const int lp = first_lp + i;
                const int page = lp < p.table_width ? bt[lp] : -1;
                const bool in_range = lp * p.page_size <= block_last_pos && (lp + 1) * p.page_size > block_lo;
                if (!in_range || page < 0 || page >= p.num_pages) continue;
                const int y = ((page * 2 + kv) * p.nkv + kvh) * p.page_size;
                tma_load_2d(stage + h * (ROWS * 128) + i * p.page_size * 128, &page_map, h * 64, y, bar);
            }
            __syncwarp();
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        if (tid == 0) {
            const unsigned long long t0 = global_timer();
            while (global_timer() - t0 < 2000000ull) { }   // let copies in flight land before the shared memory is released
            report_status(p.status, SPY_STATUS_WAIT_TIMEOUT, (int)blockIdx.x);
        }
        __syncthreads();
    }
    if (warp == 4) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)L::TMEM_COLS) : "memory");
    }
}

// One block per (sequence, head); does nothing when the token's keys lay in one split.
template <int HD>
__global__ void attention_tc_merge_kernel(const Params p)
{
    pdl_enter();
    const int seq = blockIdx.x, head = blockIdx.y, d = threadIdx.x;
    const int tok = p.q_start[seq];
    const int pos = p.positions[tok];
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int z_first = lo / p.split_keys, z_last = pos / p.split_keys;
    if (z_first == z_last) return;
    const size_t base = ((size_t)tok * p.nh + head) * p.max_splits;
    float M = -INFINITY;
    for (int z = z_first; z <= z_last; ++z) M = fmaxf(M, p.part_ml[(base + z) * 2]);
    float L = 0.f, acc = 0.f;
    for (int z = z_first; z <= z_last; ++z) {
        const float mz = p.part_ml[(base + z) * 2];
        const float f = mz == -INFINITY ? 0.f : exp2f(mz - M);
        L += p.part_ml[(base + z) * 2 + 1] * f;
        acc += p.part_o[(base + z) * HD + d] * f;
    }
    p.out[((size_t)tok * p.nh + head) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

// Floats of scratch the split mode needs for `seqs` decoding sequences.
extern "C" long long spy_attention_tc_scratch_floats(int seqs, int nh, int hd, int max_splits) { return (long long)seqs * nh * max_splits * (hd + 2); }

// Attention of a batch over its pages.  split_keys == 0: prompt portions (any mix, single tokens
// included).  split_keys > 0 (a multiple of 128): every sequence brings one token and its keys
// are cut into at most max_splits ranges of split_keys, merged through `scratch`.
extern "C" int spy_attention_tc(const void* q, long long q_row_stride, void* out, const void* pages, const int* block_table, int table_width,
                                int page_size, int num_pages, int nh, int nkv, int hd, const int* positions, const int* q_start, int tokens,
                                int seqs, int window, float scale, int split_keys, int max_splits, float* scratch, long long scratch_floats,
                                int* status, cudaStream_t stream)
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
    p.q = (const bf16*)q; p.q_stride = q_row_stride; p.out = (bf16*)out; p.pages = (const bf16*)pages; p.block_table = block_table;
    p.positions = positions; p.q_start = q_start; p.status = status; p.table_width = table_width; p.page_size = page_size;
    p.num_pages = num_pages; p.nh = nh; p.nkv = nkv; p.G = G; p.Gp = Gp; p.S = seqs; p.window = window; p.scale_log2 = scale * LOG2E;
    p.split_keys = split_keys; p.max_splits = max_splits; p.part_o = nullptr; p.part_ml = nullptr;
    if (page_size < 8 || page_size > TILE || TILE % page_size != 0)
        SPY_FAIL("attention_tc: page_size %d must be 8, 16, 32, 64 or 128 (one TMA box per page)", page_size);
    // the pages of this cache as one matrix [num_pages * 2 * nkv * page_size rows, hd]; a box is one page's rows x 64 columns
    static EncodeTiledFn encode = nullptr;
    if (encode == nullptr) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) != cudaSuccess || qr != cudaDriverEntryPointSuccess)
            SPY_FAIL("attention_tc: cuTensorMapEncodeTiled is not available from the driver");
        encode = reinterpret_cast<EncodeTiledFn>(fn);
    }
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
    static bool configured = false;
    if (!configured) {
        SPY_CUDA(cudaFuncSetAttribute(attention_tc_kernel<64, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<64>::TOTAL));
        SPY_CUDA(cudaFuncSetAttribute(attention_tc_kernel<128, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<128>::TOTAL));
        SPY_CUDA(cudaFuncSetAttribute(attention_tc_kernel<64, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<64>::TOTAL));
        SPY_CUDA(cudaFuncSetAttribute(attention_tc_kernel<128, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<128>::TOTAL));
        configured = true;
    }
    if (split_keys > 0) {
        if (tokens != seqs) SPY_FAIL("attention_tc: split mode needs one token per sequence (%d tokens, %d sequences)", tokens, seqs);
        if (split_keys % TILE != 0 || max_splits <= 0 || max_splits > 65535)
            SPY_FAIL("attention_tc: split_keys %d must be a multiple of %d and max_splits %d positive", split_keys, TILE, max_splits);
        const long long need = spy_attention_tc_scratch_floats(seqs, nh, hd, max_splits);
        if (max_splits > 1 && (scratch == nullptr || scratch_floats < need))
            SPY_FAIL("attention_tc: %lld floats of scratch are needed, %lld were given", need, scratch_floats);
        p.part_o = scratch;
        p.part_ml = scratch ? scratch + (size_t)seqs * nh * max_splits * hd : nullptr;
        if (nkv > 65535) SPY_FAIL("attention_tc: the batch exceeds the grid limits");
        dim3 grid(seqs, nkv, max_splits);
        if (hd == 64) spy_launch(attention_tc_kernel<64, true>, grid, dim3(NUM_THREADS), (size_t)Smem<64>::TOTAL, stream, page_map, p);
        else spy_launch(attention_tc_kernel<128, true>, grid, dim3(NUM_THREADS), (size_t)Smem<128>::TOTAL, stream, page_map, p);
        SPY_CHECK_LAUNCH("attention_tc (split)");
        if (max_splits > 1) {
            dim3 mgrid(seqs, nh);
            if (hd == 64) spy_launch(attention_tc_merge_kernel<64>, mgrid, dim3(64), 0, stream, p);
            else spy_launch(attention_tc_merge_kernel<128>, mgrid, dim3(128), 0, stream, p);
            SPY_CHECK_LAUNCH("attention_tc (merge)");
        }
        return 0;
    }
    const int tokens_per_block = ROWS / Gp;
    const long long blocks = (tokens + tokens_per_block - 1) / tokens_per_block + seqs;   // an upper bound without a host copy of q_start
    if (blocks > 0x7fffffffLL || nkv > 65535) SPY_FAIL("attention_tc: the batch exceeds the grid limits");
    dim3 grid((unsigned)blocks, nkv);
    if (hd == 64) spy_launch(attention_tc_kernel<64, false>, grid, dim3(NUM_THREADS), (size_t)Smem<64>::TOTAL, stream, page_map, p);
    else spy_launch(attention_tc_kernel<128, false>, grid, dim3(NUM_THREADS), (size_t)Smem<128>::TOTAL, stream, page_map, p);
    SPY_CHECK_LAUNCH("attention_tc");
    return 0;
}
