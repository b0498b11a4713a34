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
// Key/value tiles are double-buffered: the softmax warps request tile j + 1 with cp.async
// before they work on tile j.  A fifth warp allocates tensor memory and issues the MMAs.
// Every wait on an mbarrier is bounded; a wait that runs out raises the block's abort flag,
// which ends all roles, and the status word reports it.
//
// Formula and masking: spymaster2h/spyinfer src/backends/cpu/cpu_attention.cpp:89-135.  The
// reference's prefill kernel (src/backends/cuda/native/attention.cu:62-255) uses no tensor
// cores and cannot see a cached prefix.
// Limits (checked on the host): head_dim 64 or 128, G <= 16, bfloat16.
#include "common.cuh"

SPY_MODULE(spy_attention_tc)

namespace {

constexpr int ROWS = 128;          // query rows per block = UMMA M
constexpr int TILE = 128;          // keys per tile = UMMA N of the first product
constexpr int NUM_THREADS = 160;   // warps 0..3: loads, softmax, epilogue; warp 4: TMEM + MMA
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
    int table_width, page_size, num_pages, nh, nkv, G, Gp, S, window;
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
    static constexpr int HALVES = HD / 64;
    static constexpr int OPERAND_BYTES = ROWS * HD * 2;       // Q, K or V tile
    static constexpr int P_BYTES = ROWS * TILE * 2;
    static constexpr int Q_OFF = 0;
    static constexpr int K_OFF = Q_OFF + OPERAND_BYTES;       // two stages
    static constexpr int V_OFF = K_OFF + 2 * OPERAND_BYTES;   // two stages
    static constexpr int P_OFF = V_OFF + 2 * OPERAND_BYTES;
    static constexpr int BAR_OFF = P_OFF + P_BYTES;
    static constexpr int TOTAL = BAR_OFF + 128 + 1024;        // barriers, then slack to align the base to 1024
    static constexpr int TMEM_COLS = 256;                     // S: 128 columns, O: HD columns
};

template <int HD>
__global__ void __launch_bounds__(NUM_THREADS, 1) attention_tc_kernel(const Params p)
{
    using L = Smem<HD>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* bar_kv = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);   // [2] tile landed (128 arrivals)
    uint64_t* bar_s = bar_kv + 2;                                        // scores complete (MMA commit)
    uint64_t* bar_p = bar_s + 1;                                         // probabilities written (128 arrivals)
    uint64_t* bar_o = bar_p + 1;                                         // P.V complete (MMA commit)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_o + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* s_info = reinterpret_cast<int*>(tmem_slot + 2);                 // seq, first token of the block

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    const int tokens_per_block = ROWS / p.Gp;
    if (tid == 0) {
        for (int i = 0; i < 2; ++i) mbar_init(bar_kv + i, ROWS);
        mbar_init(bar_s, 1);
        mbar_init(bar_p, ROWS);
        mbar_init(bar_o, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)L::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    pdl_wait();   // everything below reads what earlier kernels wrote
    if (tid == 0) {
        int b = blockIdx.x, seq = -1, tok0 = 0;
        for (int s = 0; s < p.S; ++s) {
            const int n = p.q_start[s + 1] - p.q_start[s];
            const int blocks = (n + tokens_per_block - 1) / tokens_per_block;
            if (b < blocks) { seq = s; tok0 = p.q_start[s] + b * tokens_per_block; break; }
            b -= blocks;
        }
        s_info[0] = seq;
        s_info[1] = tok0;
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_s = tmem_base, tmem_o = tmem_base + TILE;
    const int seq = s_info[0], tok0 = s_info[1];
    const int kvh = blockIdx.y;

    int n_tiles = 0, tile_first = 0, block_lo = 0, block_last_pos = -1, tok_end = 0;
    if (seq >= 0) {
        tok_end = p.q_start[seq + 1];
        const int first_pos = p.positions[tok0];
        block_last_pos = p.positions[min(tok_end, tok0 + tokens_per_block) - 1];
        block_lo = p.window > 0 ? max(0, first_pos - p.window + 1) : 0;
        tile_first = block_lo / TILE;
        n_tiles = block_last_pos / TILE - tile_first + 1;
    }
    const uint32_t q_s = smem_u32(smem + L::Q_OFF), k_s = smem_u32(smem + L::K_OFF), v_s = smem_u32(smem + L::V_OFF),
                   p_s = smem_u32(smem + L::P_OFF);

    if (warp < 4 && seq >= 0) {
        // ---------------------------------------------------------------- loads, softmax, epilogue
        const int row = tid;                                  // this thread's query row = TMEM lane
        const int tok = tok0 + row / p.Gp, hg = row % p.Gp;
        const bool row_ok = tok < tok_end && hg < p.G;
        const int head = kvh * p.G + hg;
        const int pos = row_ok ? p.positions[tok] : -1;
        const int lo = (row_ok && p.window > 0) ? max(0, pos - p.window + 1) : 0;
        const int* bt = p.block_table + (size_t)seq * p.table_width;
        const size_t plane = (size_t)p.nkv * p.page_size * HD;

        // Q tile: this thread's row
        {
            const bf16* src = p.q + (size_t)(row_ok ? tok : 0) * p.q_stride + (size_t)head * HD;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) cp_async16(smem + L::Q_OFF + tile_offset(row, c), src + c * 8, row_ok);
        }
        auto load_tile = [&](int t) {                         // key row (tile_first + t) * TILE + tid of K and V into stage t % 2
            const int j = (tile_first + t) * TILE + tid;
            bool ok = j >= block_lo && j <= block_last_pos;
            const bf16* src = p.pages;
            if (ok) {
                const int lp = j / p.page_size;
                const int page = lp < p.table_width ? bt[lp] : -1;
                if (page < 0 || page >= p.num_pages) {
                    report_status(p.status, SPY_STATUS_BAD_PAGE, tok0);
                    ok = false;
                } else {
                    src = p.pages + (((size_t)page * 2) * p.nkv + kvh) * p.page_size * HD + (size_t)(j - lp * p.page_size) * HD;
                }
            }
            uint8_t* kd = smem + L::K_OFF + (t & 1) * L::OPERAND_BYTES;
            uint8_t* vd = smem + L::V_OFF + (t & 1) * L::OPERAND_BYTES;
#pragma unroll
            for (int c = 0; c < HD / 8; ++c) {
                cp_async16(kd + tile_offset(tid, c), src + c * 8, ok);
                cp_async16(vd + tile_offset(tid, c), src + plane + c * 8, ok);
            }
        };
        if (n_tiles > 0) load_tile(0);
        asm volatile("cp.async.wait_all;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");   // the MMA reads shared memory through the async proxy
        mbar_arrive(bar_kv + 0);

        float m_used = -INFINITY, l = 0.f;   // the maximum the probabilities are taken against, and their sum
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        bool alive = true;
        for (int t = 0; t < n_tiles && alive; ++t) {
            if (t > 0) alive = mbar_wait(bar_o, (t - 1) & 1, abort_flag);   // P.V of tile t-1 done: O, P and stage (t+1)%2 are free
            if (!alive) break;
            if (t + 1 < n_tiles) load_tile(t + 1);
            alive = mbar_wait(bar_s, t & 1, abort_flag);
            if (!alive) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int key0 = (tile_first + t) * TILE;
            // pass 1: the row's maximum over the tile
            float mx = -INFINITY;
#pragma unroll 1
            for (int c = 0; c < TILE; c += 32) {
                uint32_t r[32];
                tmem_load_32(tmem_s + lane_addr + c, r);
#pragma unroll
                for (int i = 0; i < 32; ++i) {
                    const int j = key0 + c + i;
                    const float v = (j <= pos && j >= lo) ? __uint_as_float(r[i]) * p.scale_log2 : -INFINITY;
                    mx = fmaxf(mx, v);
                }
            }
            // rescale O only when the maximum grew by more than the threshold (or from nothing)
            const float m_new = fmaxf(m_used, mx);
            const bool grow = m_new > m_used + RESCALE_THRESHOLD || (m_used == -INFINITY && m_new != -INFINITY);
            if (__any_sync(0xffffffffu, grow)) {
                const float alpha = grow ? (m_used == -INFINITY ? 0.f : fast_exp2(m_used - m_new)) : 1.f;
                if (t > 0) {
#pragma unroll 1
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t r[32];
                        tmem_load_32(tmem_o + lane_addr + c, r);
#pragma unroll
                        for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                        tmem_store_32(tmem_o + lane_addr + c, r);
                    }
                }
                if (grow) {
                    l *= alpha;
                    m_used = m_new;
                }
            }
            const float m_sub = m_used == -INFINITY ? 0.f : m_used;
            // pass 2: probabilities to shared memory as bfloat16 (A operand of P.V, K-major over the keys)
#pragma unroll 1
            for (int c = 0; c < TILE; c += 32) {
                uint32_t r[32];
                tmem_load_32(tmem_s + lane_addr + c, r);
                uint32_t packed[16];
#pragma unroll
                for (int i = 0; i < 32; i += 2) {
                    const int j = key0 + c + i;
                    const float s0 = (j <= pos && j >= lo) ? __uint_as_float(r[i]) * p.scale_log2 : -INFINITY;
                    const float s1 = (j + 1 <= pos && j + 1 >= lo) ? __uint_as_float(r[i + 1]) * p.scale_log2 : -INFINITY;
                    const float p0 = fast_exp2(s0 - m_sub), p1 = fast_exp2(s1 - m_sub);
                    l += p0 + p1;
                    packed[i / 2] = pack_bf16(p0, p1);
                }
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4)
                    *reinterpret_cast<uint4*>(smem + L::P_OFF + tile_offset(row, c / 8 + q4)) =
                        make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(bar_p);
            if (t + 1 < n_tiles) {
                asm volatile("cp.async.wait_all;" ::: "memory");
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_arrive(bar_kv + ((t + 1) & 1));
            }
        }
        // ---- epilogue: O / l
        if (alive && n_tiles > 0) alive = mbar_wait(bar_o, (n_tiles - 1) & 1, abort_flag);
        if (alive && n_tiles > 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = l > 0.f ? 1.f / l : 0.f;
            bf16* dst = p.out + ((size_t)(row_ok ? tok : 0) * p.nh + head) * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t r[32];
                tmem_load_32(tmem_o + lane_addr + c, r);
                if (row_ok) {
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
        }
    } else if (warp == 4 && seq >= 0) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc_qk = instr_desc(TILE, false), idesc_pv = instr_desc(HD, true);
            auto issue_qk = [&](int t) {
                const uint32_t kb = k_s + (t & 1) * L::OPERAND_BYTES;
#pragma unroll
                for (int s = 0; s < HD / 16; ++s) {
                    const uint32_t off = (s >> 2) * (ROWS * 128) + (s & 3) * 32;   // 64-element half, then 32 bytes per 16 elements
                    umma(tmem_s, desc_k_major(q_s + off), desc_k_major(kb + off), idesc_qk, s > 0 ? 1u : 0u);
                }
                umma_commit(bar_s);
            };
            bool ok = n_tiles > 0 && mbar_wait(bar_kv + 0, 0, abort_flag);
            if (ok) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_qk(0);
            }
            for (int t = 0; t < n_tiles && ok; ++t) {
                ok = mbar_wait(bar_p, t & 1, abort_flag);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t vb = v_s + (t & 1) * L::OPERAND_BYTES;
#pragma unroll
                for (int s = 0; s < TILE / 16; ++s) {
                    const uint32_t a_off = (s >> 2) * (ROWS * 128) + (s & 3) * 32;   // P: 16 keys = 32 bytes along its rows
                    const uint32_t b_off = s * 16 * 128;                             // V: 16 key rows of 128 bytes
                    umma(tmem_o, desc_k_major(p_s + a_off), desc_mn_major(vb + b_off, ROWS * 128), idesc_pv, (t > 0 || s > 0) ? 1u : 0u);
                }
                umma_commit(bar_o);
                if (t + 1 < n_tiles) {
                    ok = mbar_wait(bar_kv + ((t + 1) & 1), ((t + 1) >> 1) & 1, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    issue_qk(t + 1);
                }
            }
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

}  // namespace

// Attention of a batch of prompt portions (any mix, single tokens included) over its pages.
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
    p.q = (const bf16*)q; p.q_stride = q_row_stride; p.out = (bf16*)out; p.pages = (const bf16*)pages; p.block_table = block_table;
    p.positions = positions; p.q_start = q_start; p.status = status; p.table_width = table_width; p.page_size = page_size;
    p.num_pages = num_pages; p.nh = nh; p.nkv = nkv; p.G = G; p.Gp = Gp; p.S = seqs; p.window = window; p.scale_log2 = scale * LOG2E;
    const int tokens_per_block = ROWS / Gp;
    const long long blocks = (tokens + tokens_per_block - 1) / tokens_per_block + seqs;   // an upper bound without a host copy of q_start
    if (blocks > 0x7fffffffLL || nkv > 65535) SPY_FAIL("attention_tc: the batch exceeds the grid limits");
    dim3 grid((unsigned)blocks, nkv);
    static bool configured = false;
    if (!configured) {
        SPY_CUDA(cudaFuncSetAttribute(attention_tc_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<64>::TOTAL));
        SPY_CUDA(cudaFuncSetAttribute(attention_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem<128>::TOTAL));
        configured = true;
    }
    if (hd == 64) spy_launch(attention_tc_kernel<64>, grid, dim3(NUM_THREADS), (size_t)Smem<64>::TOTAL, stream, p);
    else spy_launch(attention_tc_kernel<128>, grid, dim3(NUM_THREADS), (size_t)Smem<128>::TOTAL, stream, p);
    SPY_CHECK_LAUNCH("attention_tc");
    return 0;
}
