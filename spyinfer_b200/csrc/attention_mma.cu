// bfloat16 attention over the paged cache on the tensor cores (mma.sync m16n8k16), keys and
// values streamed from the pages with cp.async in the order of the instruction's operand
// registers (in split mode every thread copies its own 16-byte pieces into a private ring in
// shared memory, an asynchronous extension of its registers).  One warp owns a tile of 16 rows = the G query
// heads of one key/value head for 16 / Gp consecutive tokens of one sequence (Gp = G rounded
// up to a power of two), so every key and value row is read once for all G heads.
//
// Two launch modes:
//   tiles  (any batch): a block's eight warps take eight consecutive token tiles of a sequence
//          and share the keys and values, which go through tiles of 64 keys in shared memory;
//          each warp writes its output rows directly.
//   split  (every sequence brings exactly one token: decoding): grid (sequence, kv head,
//          split); split z covers keys [z * split_keys, (z + 1) * split_keys); the four warps
//          share that range and merge in shared memory; when a row's keys span more than one
//          split, partial (max, sum, unnormalised output) go to scratch and a second kernel
//          merges them in split order.
//
// The element order inside a 32-element chunk of head_dim is permuted identically for
// queries and keys (a dot product does not care), which is what lets a thread's 16-byte
// load be its own operand fragment.  Softmax in 32-bit with exp2f on pre-scaled scores;
// probabilities are rounded to bfloat16 for the second product, which accumulates in
// 32-bit.  Formula and masking as in spymaster2h/spyinfer
// src/backends/cpu/cpu_attention.cpp:89-135; this replaces its
// paged_attention_decode_kernel and flash prefill kernel
// (src/backends/cuda/native/attention.cu:62-370), which use no tensor cores, read the cache
// once per query head, and cannot handle a prefix or a mixed batch.
//
// Limits (checked on the host; other sizes go to the plain kernel): head_dim 64 or 128,
// G <= 16, bfloat16 queries and cache.
#include "common.cuh"

SPY_MODULE(spy_attention_mma)

namespace {

constexpr int WARPS = 4;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void mma_bf16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1)
{
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi)
{
    __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&t);
}

__device__ __forceinline__ float fast_exp2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));   // exp2(-inf) = 0
    return y;
}

__device__ __forceinline__ uint4 load16(const bf16* p) { return *reinterpret_cast<const uint4*>(p); }

__device__ __forceinline__ uint32_t word(const uint4& v, int i) { return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w)); }

struct Params {
    const bf16* q;
    long long q_stride;
    bf16* out;                 // [T, nh * HD]
    const bf16* pages;         // [num_pages][2][nkv][page_size][HD]
    const int* block_table;    // [S, table_width]
    const int* positions;      // [T]
    const int* q_start;        // [S + 1]
    float* part_o;             // [T][nh][max_splits][HD]     (split mode)
    float* part_ml;            // [T][nh][max_splits][2]
    int* status;
    int table_width, page_size, num_pages, nh, nkv, G, Gp, S, window, split_keys, max_splits;
    float scale_log2;
};

// State of one warp's 16-row tile while it walks a range of keys.
template <int HD> struct TileState {
    float o[HD / 64][8][4];   // output accumulators: [d set of 64][n-tile][c0..c3]
    float m[2], l[2];         // running max (log2 domain) and this thread's share of the sum, rows g and g + 8
};

constexpr int RING = 3;   // stages of the per-thread copy ring

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* src, bool valid)
{
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 bytes are filled with zeros
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Looks a key's page up: in `bt_s` (shared copy of the block table from logical page
// `bt_first` on) when it is given, else in the global table.
__device__ __forceinline__ int page_of(const Params& p, const int* bt, const int* bt_s, int bt_first, int lp)
{
    if (bt_s != nullptr) return bt_s[lp - bt_first];
    return lp < p.table_width ? bt[lp] : -1;
}

// The arithmetic on one group of 16 keys [kb, kb + 16) for one 16-row tile: scores, mask, online
// softmax, output update.  ld_k(tile, c) returns this thread's 16 bytes of K for key
// kb + 8 tile + g, chunk c; ld_v(i, ds) its 16 bytes of V for key kb + 2 t4 + (i & 1) + 8 (i >> 1),
// column set ds.  Groups that every used row sees whole ([all_lo, all_hi]) skip the masking;
// the running output is rescaled only when some row's maximum grew.
template <int HD, typename LoadK, typename LoadV>
__device__ __forceinline__ void process_group(const Params& p, const uint4 (&qf)[2][HD / 32], const int (&row_pos)[2], const int (&row_lo)[2],
                                              int key_lo, int key_hi, int all_lo, int all_hi, int kb, TileState<HD>& st, LoadK ld_k, LoadV ld_v)
{
    const int lane = threadIdx.x & 31, t4 = lane & 3;
    constexpr int KC = HD / 32;   // 32-element chunks of head_dim
    constexpr int DS = HD / 64;   // sets of 64 output columns
    // ---- scores of 16 rows x 16 keys (two accumulators per key tile keep four chains in flight)
    float s[2][4], s2[2][4];
#pragma unroll
    for (int tile = 0; tile < 2; ++tile)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[tile][e] = s2[tile][e] = 0.f;
#pragma unroll
    for (int c = 0; c < KC; ++c) {
        const uint4 k0 = ld_k(0, c), k1 = ld_k(1, c);
        mma_bf16(s[0], qf[0][c].x, qf[1][c].x, qf[0][c].y, qf[1][c].y, k0.x, k0.y);
        mma_bf16(s[1], qf[0][c].x, qf[1][c].x, qf[0][c].y, qf[1][c].y, k1.x, k1.y);
        mma_bf16(s2[0], qf[0][c].z, qf[1][c].z, qf[0][c].w, qf[1][c].w, k0.z, k0.w);
        mma_bf16(s2[1], qf[0][c].z, qf[1][c].z, qf[0][c].w, qf[1][c].w, k1.z, k1.w);
    }
#pragma unroll
    for (int tile = 0; tile < 2; ++tile)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[tile][e] += s2[tile][e];
    // ---- scale, mask (only in groups that some row cannot see whole), running max
    const bool whole = kb >= all_lo && kb + 15 <= all_hi;   // uniform over the warp
    float mx[2] = {-INFINITY, -INFINITY};
    if (whole) {
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                s[tile][e] *= p.scale_log2;
                mx[e >> 1] = fmaxf(mx[e >> 1], s[tile][e]);
            }
    } else {
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;                              // c0, c1: row g; c2, c3: row g + 8
                const int j = kb + tile * 8 + 2 * t4 + (e & 1);
                const bool ok = j <= row_pos[r] && j >= row_lo[r] && j >= key_lo && j <= key_hi;
                const float v = ok ? s[tile][e] * p.scale_log2 : -INFINITY;
                s[tile][e] = v;
                mx[r] = fmaxf(mx[r], v);
            }
    }
    bool grew = false;
    float m_new[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        m_new[r] = fmaxf(st.m[r], mx[r]);
        grew = grew || m_new[r] != st.m[r];
    }
    if (__any_sync(0xffffffffu, grew)) {
        float alpha[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            alpha[r] = m_new[r] == -INFINITY ? 1.f : fast_exp2(st.m[r] - m_new[r]);   // st.m = -inf gives 0
            st.m[r] = m_new[r];
            st.l[r] *= alpha[r];
        }
#pragma unroll
        for (int ds = 0; ds < DS; ++ds)
#pragma unroll
            for (int jt = 0; jt < 8; ++jt) {
                st.o[ds][jt][0] *= alpha[0];
                st.o[ds][jt][1] *= alpha[0];
                st.o[ds][jt][2] *= alpha[1];
                st.o[ds][jt][3] *= alpha[1];
            }
    }
    // ---- probabilities
    uint32_t pa[4];   // A fragment of P: a0 (row g, keys 2t4..), a1 (row g+8), a2 (row g, keys 8+2t4..), a3 (row g+8)
    {
        float pr[2][4];
        // a row that has seen no key yet has max -inf: its scores are -inf too and must give 0, not NaN
        const float m0 = st.m[0] == -INFINITY ? 0.f : st.m[0], m1 = st.m[1] == -INFINITY ? 0.f : st.m[1];
#pragma unroll
        for (int tile = 0; tile < 2; ++tile)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int r = e >> 1;
                const float v = fast_exp2(s[tile][e] - (r == 0 ? m0 : m1));
                pr[tile][e] = v;
                st.l[r] += v;
            }
        pa[0] = pack_bf16(pr[0][0], pr[0][1]);
        pa[1] = pack_bf16(pr[0][2], pr[0][3]);
        pa[2] = pack_bf16(pr[1][0], pr[1][1]);
        pa[3] = pack_bf16(pr[1][2], pr[1][3]);
    }
    // ---- O += P V
#pragma unroll
    for (int ds = 0; ds < DS; ++ds) {
        uint4 vf[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) vf[i] = ld_v(i, ds);
#pragma unroll
        for (int jt = 0; jt < 8; ++jt) {
            const uint32_t sel = (jt & 1) ? 0x7632u : 0x5410u;   // upper or lower halves of the two words
            const uint32_t b0 = __byte_perm(word(vf[0], jt >> 1), word(vf[1], jt >> 1), sel);
            const uint32_t b1 = __byte_perm(word(vf[2], jt >> 1), word(vf[3], jt >> 1), sel);
            mma_bf16(st.o[ds][jt], pa[0], pa[1], pa[2], pa[3], b0, b1);
        }
    }
}

// The keys every used row of a warp's tile can see, as one range (uniform over the warp).
__device__ __forceinline__ void common_range(const int (&row_pos)[2], const int (&row_lo)[2], int key_lo, int key_hi, int& all_lo, int& all_hi)
{
    all_lo = key_lo;
    all_hi = key_hi;
#pragma unroll
    for (int r = 0; r < 2; ++r)
        if (row_pos[r] >= 0) {
            all_lo = max(all_lo, row_lo[r]);
            all_hi = min(all_hi, row_pos[r]);
        }
    all_lo = __reduce_max_sync(0xffffffffu, all_lo);
    all_hi = __reduce_min_sync(0xffffffffu, all_hi);
}

// Walks keys [key_lo, key_hi] (inclusive, absolute positions) for one tile.
// row_pos / row_lo: last and first visible key of rows g and g + 8 (row_pos < 0: row unused).
// Every thread copies exactly the 16-byte pieces it will use itself (its operand fragments
// of 16 keys: 8 pieces of K, 8 of V for head_dim 128) into its own slots of a ring in shared
// memory with cp.async, RING - 1 groups of 16 keys ahead of the one it computes on; no
// thread reads another thread's slots, so the ring needs no barrier.
// ring: [RING][2 * HD / 16 pieces][blockDim.x] of 16 bytes.
// PAGE16: the page size is a multiple of 16, so the 16 keys of a group share one page and
// one block-table lookup serves the whole group.
template <int HD, bool PAGE16>
__device__ __forceinline__ void walk_keys(const Params& p, const int* bt, const int* bt_s, int bt_first, int kvh, const uint4 (&qf)[2][HD / 32],
                                          const int (&row_pos)[2], const int (&row_lo)[2], int key_lo, int key_hi, TileState<HD>& st,
                                          uint4* ring, int tok_for_status)
{
    const int lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    constexpr int KC = HD / 32;   // 32-element chunks of head_dim
    constexpr int DS = HD / 64;   // sets of 64 output columns
    constexpr int PIECES = 2 * KC + 4 * DS;
    const int nthreads = blockDim.x;
    const int kb_first = key_lo & ~15;
    const int n_iter = (key_hi - kb_first) / 16 + 1;
    const size_t plane = (size_t)p.nkv * p.page_size * HD;   // elements from a page's K plane to its V plane
    int all_lo, all_hi;
    common_range(row_pos, row_lo, key_lo, key_hi, all_lo, all_hi);

    auto page_base = [&](int lp) -> const bf16* {   // K plane of this kv head in logical page lp, or null
        const int page = page_of(p, bt, bt_s, bt_first, lp);
        if (page < 0 || page >= p.num_pages) {
            report_status(p.status, SPY_STATUS_BAD_PAGE, tok_for_status);
            return nullptr;
        }
        return p.pages + (((size_t)page * 2) * p.nkv + kvh) * p.page_size * HD;
    };

    auto issue = [&](int it) {
        if (it < n_iter) {
            const int kb = kb_first + it * 16;
            uint4* slot = ring + ((size_t)(it % RING) * PIECES) * nthreads + threadIdx.x;
            const bf16* group_base = nullptr;
            int group_slot = 0;
            if constexpr (PAGE16) {
                const int lp = kb / p.page_size;
                group_base = page_base(lp);
                group_slot = kb - lp * p.page_size;
            }
#pragma unroll
            for (int tile = 0; tile < 2; ++tile) {
                const int j = kb + tile * 8 + g;
                bool ok = j >= key_lo && j <= key_hi;
                const bf16* row = p.pages;
                if constexpr (PAGE16) {
                    ok = ok && group_base != nullptr;
                    if (ok) row = group_base + (size_t)(group_slot + tile * 8 + g) * HD;
                } else if (ok) {
                    const int lp = j / p.page_size;
                    const bf16* base = page_base(lp);
                    ok = base != nullptr;
                    if (ok) row = base + (size_t)(j - lp * p.page_size) * HD;
                }
#pragma unroll
                for (int c = 0; c < KC; ++c) cp_async16(slot + (size_t)(tile * KC + c) * nthreads, row + c * 32 + t4 * 8, ok);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int off = 2 * t4 + (i & 1) + (i >> 1) * 8;
                const int j = kb + off;
                bool ok = j >= key_lo && j <= key_hi;
                const bf16* row = p.pages;
                if constexpr (PAGE16) {
                    ok = ok && group_base != nullptr;
                    if (ok) row = group_base + plane + (size_t)(group_slot + off) * HD;
                } else if (ok) {
                    const int lp = j / p.page_size;
                    const bf16* base = page_base(lp);
                    ok = base != nullptr;
                    if (ok) row = base + plane + (size_t)(j - lp * p.page_size) * HD;
                }
#pragma unroll
                for (int ds = 0; ds < DS; ++ds) cp_async16(slot + (size_t)(2 * KC + i * DS + ds) * nthreads, row + ds * 64 + g * 8, ok);
            }
        }
        cp_async_commit();   // an empty group keeps the count of groups in step with the iterations
    };

#pragma unroll
    for (int s = 0; s < RING - 1; ++s) issue(s);
    for (int it = 0; it < n_iter; ++it) {
        issue(it + RING - 1);
        cp_async_wait<RING - 1>();
        const int kb = kb_first + it * 16;
        const uint4* slot = ring + ((size_t)(it % RING) * PIECES) * nthreads + threadIdx.x;
        process_group<HD>(p, qf, row_pos, row_lo, key_lo, key_hi, all_lo, all_hi, kb, st,
                          [&](int tile, int c) { return slot[(size_t)(tile * KC + c) * nthreads]; },
                          [&](int i, int ds) { return slot[(size_t)(2 * KC + i * DS + ds) * nthreads]; });
    }
    cp_async_wait<0>();
}

template <int HD> __device__ __forceinline__ void init_state(TileState<HD>& st)
{
#pragma unroll
    for (int ds = 0; ds < HD / 64; ++ds)
#pragma unroll
        for (int jt = 0; jt < 8; ++jt) st.o[ds][jt][0] = st.o[ds][jt][1] = st.o[ds][jt][2] = st.o[ds][jt][3] = 0.f;
    st.m[0] = st.m[1] = -INFINITY;
    st.l[0] = st.l[1] = 0.f;
}

// Loads the query fragments of rows g and g + 8 (zeros for unused rows).
template <int HD>
__device__ __forceinline__ void load_q(const Params& p, int kvh, int tok0, int tok_end, uint4 (&qf)[2][HD / 32], int (&row_tok)[2], int (&row_head)[2])
{
    const int lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int row = g + 8 * r;
        const int tok = tok0 + row / p.Gp, hg = row % p.Gp;
        const bool ok = tok < tok_end && hg < p.G;
        row_tok[r] = ok ? tok : -1;
        row_head[r] = kvh * p.G + hg;
        const bf16* src = p.q + (size_t)(ok ? tok : 0) * p.q_stride + (size_t)row_head[r] * HD;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) qf[r][c] = ok ? load16(src + c * 32 + t4 * 8) : make_uint4(0, 0, 0, 0);
    }
}

// The thread's share of a finished tile: rows g and g + 8, 16 consecutive columns per set of 64.
template <int HD>
__device__ __forceinline__ void store_rows(const Params& p, const TileState<HD>& st, const int (&row_tok)[2], const int (&row_head)[2])
{
    const int lane = threadIdx.x & 31, t4 = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = st.l[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        if (row_tok[r] < 0) continue;
        const float inv = l > 0.f ? 1.f / l : 0.f;
        bf16* dst = p.out + ((size_t)row_tok[r] * p.nh + row_head[r]) * HD;
#pragma unroll
        for (int ds = 0; ds < HD / 64; ++ds) {
            // column n of n-tile jt holds d = ds * 64 + n * 8 + jt; this thread has n = 2 t4 (c0 / c2) and 2 t4 + 1 (c1 / c3)
            uint4 lo, hi;
            const int e = 2 * r;
            lo.x = pack_bf16(st.o[ds][0][e] * inv, st.o[ds][1][e] * inv);
            lo.y = pack_bf16(st.o[ds][2][e] * inv, st.o[ds][3][e] * inv);
            lo.z = pack_bf16(st.o[ds][4][e] * inv, st.o[ds][5][e] * inv);
            lo.w = pack_bf16(st.o[ds][6][e] * inv, st.o[ds][7][e] * inv);
            hi.x = pack_bf16(st.o[ds][0][e + 1] * inv, st.o[ds][1][e + 1] * inv);
            hi.y = pack_bf16(st.o[ds][2][e + 1] * inv, st.o[ds][3][e + 1] * inv);
            hi.z = pack_bf16(st.o[ds][4][e + 1] * inv, st.o[ds][5][e + 1] * inv);
            hi.w = pack_bf16(st.o[ds][6][e + 1] * inv, st.o[ds][7][e + 1] * inv);
            *reinterpret_cast<uint4*>(dst + ds * 64 + 16 * t4) = lo;
            *reinterpret_cast<uint4*>(dst + ds * 64 + 16 * t4 + 8) = hi;
        }
    }
}

// ---- tiles mode ------------------------------------------------------------------------------
// A block's warps take consecutive token tiles of one sequence and walk the keys together:
// tiles of 64 keys go through a three-stage ring in shared memory (cp.async by all threads,
// one barrier per tile) and every warp reads its operand fragments from them.  Rows of the
// shared tiles are 16-byte-chunk swizzled so that those reads hit distinct banks:
//   K rows: chunk ^ (((row & 1) << 2) | ((row >> 1) & 3))   (a warp reads 8 consecutive rows x 4 chunks)
//   V rows: chunk ^ (row & 7)                               (a warp reads rows 2 apart x 8 chunks)
constexpr int TILE_KEYS = 64;
constexpr int TILE_STAGES = 3;

__device__ __forceinline__ int swz_k(int row) { return ((row & 1) << 2) | ((row >> 1) & 3); }
__device__ __forceinline__ int swz_v(int row) { return row & 7; }

template <int HD, int NWARPS>
__global__ void __launch_bounds__(NWARPS * 32, NWARPS <= 4 ? 2 : 1) attention_tiles_kernel(const Params p)
{
    extern __shared__ uint4 tile_smem[];   // [TILE_STAGES][2 (K, V)][TILE_KEYS][HD / 8] chunks of 16 bytes
    __shared__ int s_seq, s_tok0;
    pdl_enter();
    constexpr int CPR = HD / 8;                        // 16-byte chunks per row
    constexpr int STAGE_CHUNKS = 2 * TILE_KEYS * CPR;
    const int tokens_per_tile = 16 / p.Gp, tokens_per_block = NWARPS * tokens_per_tile;
    if (threadIdx.x == 0) {
        // block b of the grid -> (sequence, token block within it)
        int b = blockIdx.x, seq = -1, tok0 = 0;
        for (int s = 0; s < p.S; ++s) {
            const int n = p.q_start[s + 1] - p.q_start[s];
            const int blocks = (n + tokens_per_block - 1) / tokens_per_block;
            if (b < blocks) { seq = s; tok0 = p.q_start[s] + b * tokens_per_block; break; }
            b -= blocks;
        }
        s_seq = seq;
        s_tok0 = tok0;
    }
    __syncthreads();
    const int seq = s_seq;
    if (seq < 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3, kvh = blockIdx.y;
    const int tok_end = p.q_start[seq + 1];
    const int block_tok0 = s_tok0;
    const int* bt = p.block_table + (size_t)seq * p.table_width;
    const size_t plane = (size_t)p.nkv * p.page_size * HD;

    // the block's key range: its tokens are consecutive positions of one sequence
    const int block_first_pos = p.positions[block_tok0];
    const int block_last_pos = p.positions[min(tok_end, block_tok0 + tokens_per_block) - 1];
    const int block_lo = p.window > 0 ? max(0, block_first_pos - p.window + 1) : 0;
    const int tile_first = block_lo / TILE_KEYS;
    const int n_tiles = block_last_pos / TILE_KEYS - tile_first + 1;

    // this warp's tile
    const int tok0 = block_tok0 + warp * tokens_per_tile;
    const bool active = tok0 < tok_end;
    uint4 qf[2][HD / 32];
    int row_tok[2] = {-1, -1}, row_head[2] = {0, 0}, row_pos[2] = {-1, -1}, row_lo[2] = {0, 0};
    int key_lo = 0, key_hi = -1, all_lo = 0, all_hi = -1;
    if (active) {
        load_q<HD>(p, kvh, tok0, tok_end, qf, row_tok, row_head);
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            row_pos[r] = row_tok[r] >= 0 ? p.positions[row_tok[r]] : -1;
            row_lo[r] = (row_tok[r] >= 0 && p.window > 0) ? max(0, row_pos[r] - p.window + 1) : 0;
        }
        key_lo = p.window > 0 ? max(0, p.positions[tok0] - p.window + 1) : 0;
        key_hi = p.positions[min(tok_end, tok0 + tokens_per_tile) - 1];
        common_range(row_pos, row_lo, key_lo, key_hi, all_lo, all_hi);
    }
    TileState<HD> st;
    init_state<HD>(st);

    auto issue = [&](int t) {
        if (t < n_tiles) {
            uint4* stage = tile_smem + (size_t)(t % TILE_STAGES) * STAGE_CHUNKS;
            const int key0 = (tile_first + t) * TILE_KEYS;
            for (int idx = threadIdx.x; idx < STAGE_CHUNKS; idx += NWARPS * 32) {
                const int kv = idx / (TILE_KEYS * CPR);
                const int row = (idx / CPR) % TILE_KEYS, chunk = idx % CPR;
                const int j = key0 + row;
                bool ok = j >= block_lo && j <= block_last_pos;
                const bf16* src = p.pages;
                if (ok) {
                    const int lp = j / p.page_size;
                    const int page = lp < p.table_width ? bt[lp] : -1;
                    if (page < 0 || page >= p.num_pages) {
                        report_status(p.status, SPY_STATUS_BAD_PAGE, block_tok0);
                        ok = false;
                    } else {
                        src = p.pages + (((size_t)page * 2) * p.nkv + kvh) * p.page_size * HD + kv * plane + (size_t)(j - lp * p.page_size) * HD +
                              chunk * 8;
                    }
                }
                const int phys = chunk ^ (kv == 0 ? swz_k(row) : swz_v(row));
                cp_async16(stage + (size_t)kv * TILE_KEYS * CPR + (size_t)row * CPR + phys, src, ok);
            }
        }
        cp_async_commit();
    };

    // this thread's fragment addresses inside a group of 16 keys: K row g (+ 8 tile), chunk
    // 4 c + t4; V row 2 t4 + (i & 1) (+ 8 (i >> 1)), chunk 8 ds + g; the swizzle of a row depends
    // only on its low three bits, which the group's and the tile's offsets (multiples of 8) leave alone
    const int k_off = g * CPR, v_off = 2 * t4 * CPR;
    int k_chunk[HD / 32], v_chunk[2][HD / 64];
#pragma unroll
    for (int c = 0; c < HD / 32; ++c) k_chunk[c] = (c * 4 + t4) ^ swz_k(g);
#pragma unroll
    for (int o = 0; o < 2; ++o)
#pragma unroll
        for (int ds = 0; ds < HD / 64; ++ds) v_chunk[o][ds] = (ds * 8 + g) ^ swz_v(2 * t4 + o);

    issue(0);
    issue(1);
    for (int t = 0; t < n_tiles; ++t) {
        cp_async_wait<1>();      // tile t has landed (tile t + 1 may still be in flight)
        __syncthreads();         // ... for every thread; and every warp is done with tile t - 1
        issue(t + 2);            // into the stage that held tile t - 1
        if (!active) continue;
        const uint4* ks = tile_smem + (size_t)(t % TILE_STAGES) * STAGE_CHUNKS + k_off;
        const uint4* vs = tile_smem + (size_t)(t % TILE_STAGES) * STAGE_CHUNKS + TILE_KEYS * CPR + v_off;
        const int key0 = (tile_first + t) * TILE_KEYS;
#pragma unroll 1
        for (int kk = 0; kk < TILE_KEYS / 16; ++kk) {
            const int kb = key0 + kk * 16;
            if (kb > key_hi || kb + 15 < key_lo) continue;   // no row of this warp sees the group
            const uint4* kg = ks + kk * 16 * CPR;
            const uint4* vg = vs + kk * 16 * CPR;
            process_group<HD>(p, qf, row_pos, row_lo, key_lo, key_hi, all_lo, all_hi, kb, st,
                              [&](int tile, int c) { return kg[tile * 8 * CPR + k_chunk[c]]; },
                              [&](int i, int ds) { return vg[((i & 1) + (i >> 1) * 8) * CPR + v_chunk[i & 1][ds]]; });
        }
    }
    cp_async_wait<0>();
    if (active) store_rows<HD>(p, st, row_tok, row_head);
}

// ---- split mode -------------------------------------------------------------------------------
template <int HD>
__global__ void __launch_bounds__(WARPS * 32, 2) attention_split_kernel(const Params p)
{
    // shared memory: the copy ring, then this split's slice of the block table; after the walk
    // the ring's space is reused for the merge: [WARPS][16][HD] outputs, then [WARPS][16][2] (m, l)
    extern __shared__ uint4 ring_smem[];
    pdl_enter();
    constexpr int PIECES = 2 * (HD / 32) + 4 * (HD / 64);
    float* s_o = reinterpret_cast<float*>(ring_smem);
    float* s_ml = s_o + WARPS * 16 * HD;
    int* bt_s = reinterpret_cast<int*>(ring_smem + (size_t)RING * PIECES * WARPS * 32);
    const int seq = blockIdx.x, kvh = blockIdx.y, z = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int tok = p.q_start[seq];
    const int pos = p.positions[tok];
    const int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
    const int z_first = lo / p.split_keys, z_last = pos / p.split_keys;
    if (z < z_first || z > z_last) return;
    const int key_lo = max(lo, z * p.split_keys), key_hi = min(pos, (z + 1) * p.split_keys - 1);
    const int* bt = p.block_table + (size_t)seq * p.table_width;
    const int bt_first = key_lo / p.page_size, bt_last = key_hi / p.page_size;
    for (int i = bt_first + threadIdx.x; i <= bt_last; i += WARPS * 32) bt_s[i - bt_first] = i < p.table_width ? bt[i] : -1;

    uint4 qf[2][HD / 32];
    int row_tok[2], row_head[2], row_pos[2], row_lo[2];
    load_q<HD>(p, kvh, tok, tok + 1, qf, row_tok, row_head);
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        row_pos[r] = row_tok[r] >= 0 ? pos : -1;
        row_lo[r] = lo;
    }
    __syncthreads();   // the block table slice is in shared memory
    // the four warps share the split: warp w takes its w-th quarter
    const int sub = p.split_keys / WARPS;
    const int w_lo = max(key_lo, z * p.split_keys + warp * sub), w_hi = min(key_hi, z * p.split_keys + (warp + 1) * sub - 1);
    TileState<HD> st;
    init_state<HD>(st);
    if (w_lo <= w_hi) {
        if (p.page_size % 16 == 0) walk_keys<HD, true>(p, bt, bt_s, bt_first, kvh, qf, row_pos, row_lo, w_lo, w_hi, st, ring_smem, tok);
        else walk_keys<HD, false>(p, bt, bt_s, bt_first, kvh, qf, row_pos, row_lo, w_lo, w_hi, st, ring_smem, tok);
    }
    __syncthreads();   // every warp is done with the ring before it is reused

    // ---- merge the four warps in shared memory
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        float l = st.l[r];
        l += __shfl_xor_sync(0xffffffffu, l, 1);
        l += __shfl_xor_sync(0xffffffffu, l, 2);
        const int row = g + 8 * r;
        if (t4 == 0) {
            s_ml[(warp * 16 + row) * 2] = st.m[r];
            s_ml[(warp * 16 + row) * 2 + 1] = l;
        }
        float* orow = s_o + ((size_t)warp * 16 + row) * HD;
#pragma unroll
        for (int ds = 0; ds < HD / 64; ++ds)
#pragma unroll
            for (int jt = 0; jt < 8; ++jt) {
                orow[ds * 64 + (2 * t4) * 8 + jt] = st.o[ds][jt][2 * r];
                orow[ds * 64 + (2 * t4 + 1) * 8 + jt] = st.o[ds][jt][2 * r + 1];
            }
    }
    __syncthreads();
    const bool direct = z_first == z_last;
    for (int idx = threadIdx.x; idx < p.Gp * HD; idx += WARPS * 32) {
        const int row = idx / HD, d = idx - row * HD;   // row = head within the group (one token)
        if (row >= p.G) continue;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) M = fmaxf(M, s_ml[(w * 16 + row) * 2]);
        float L = 0.f, acc = 0.f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            const float mw = s_ml[(w * 16 + row) * 2];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L += s_ml[(w * 16 + row) * 2 + 1] * f;
            acc += s_o[((size_t)w * 16 + row) * HD + d] * f;
        }
        const int head = kvh * p.G + row;
        if (direct) {
            p.out[((size_t)tok * p.nh + head) * HD + d] = __float2bfloat16_rn(L > 0.f ? acc / L : 0.f);
        } else {
            const size_t slot = ((size_t)tok * p.nh + head) * p.max_splits + z;
            p.part_o[slot * HD + d] = acc;
            if (d == 0) {
                p.part_ml[slot * 2] = M;
                p.part_ml[slot * 2 + 1] = L;
            }
        }
    }
}

// One block per (token, head); does nothing when the row's keys lay in one split.
template <int HD>
__global__ void attention_merge_kernel(const Params p)
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

}  // namespace

// Floats of scratch the split mode needs for `seqs` decoding sequences.
extern "C" long long spy_attention_mma_scratch_floats(int seqs, int nh, int hd, int max_splits)
{
    return (long long)seqs * nh * max_splits * (hd + 2);
}

// mode 0: tiles (any batch; `tokens` and q_start describe it).  mode 1: split (every sequence
// brings one token); scratch must hold spy_attention_mma_scratch_floats(S, nh, hd, max_splits)
// floats; max_splits >= ceil(longest context / split_keys); split_keys a multiple of 64.
extern "C" int spy_attention_mma(const void* q, long long q_row_stride, void* out, const void* pages, const int* block_table, int table_width,
                                 int page_size, int num_pages, int nh, int nkv, int hd, const int* positions, const int* q_start, int tokens,
                                 int seqs, int window, float scale, int mode, int split_keys, int max_splits, float* scratch,
                                 long long scratch_floats, int* status, cudaStream_t stream)
{
    if (tokens <= 0 || seqs <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) SPY_FAIL("attention_mma: %d query heads do not group over %d key/value heads", nh, nkv);
    const int G = nh / nkv;
    if (G > 16) SPY_FAIL("attention_mma: %d query heads per key/value head exceed 16", G);
    if (hd != 64 && hd != 128) SPY_FAIL("attention_mma: head_dim %d is not 64 or 128", hd);
    if (q_row_stride % 8 != 0 || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(pages) & 15) ||
        (reinterpret_cast<uintptr_t>(out) & 15))
        SPY_FAIL("attention_mma: queries, pages and output must be 16-byte aligned with rows a multiple of 8 elements");
    if (page_size <= 0 || num_pages <= 0 || table_width <= 0) SPY_FAIL("attention_mma: page_size, num_pages and table_width must be positive");
    if (window < 0) SPY_FAIL("attention_mma: window %d must be 0 (none) or positive", window);
    int Gp = 1;
    while (Gp < G) Gp *= 2;
    Params p;
    p.q = (const bf16*)q; p.q_stride = q_row_stride; p.out = (bf16*)out; p.pages = (const bf16*)pages; p.block_table = block_table;
    p.positions = positions; p.q_start = q_start; p.part_o = nullptr; p.part_ml = nullptr; p.status = status;
    p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages; p.nh = nh; p.nkv = nkv; p.G = G; p.Gp = Gp; p.S = seqs;
    p.window = window; p.split_keys = split_keys; p.max_splits = max_splits; p.scale_log2 = scale * LOG2E;
    if (mode == 0) {
#ifndef SPY_TILES_WARPS
#define SPY_TILES_WARPS 8
#endif
        constexpr int TW = SPY_TILES_WARPS;   // warps of a tiles-mode block
        const int tokens_per_block = TW * (16 / Gp);
        // every sequence rounds up to whole blocks: an upper bound that needs no host copy of q_start
        const long long blocks = (tokens + tokens_per_block - 1) / tokens_per_block + seqs;
        if (blocks > 0x7fffffffLL || nkv > 65535) SPY_FAIL("attention_mma: the batch exceeds the grid limits");
        dim3 grid((unsigned)blocks, nkv);
        const size_t tile_bytes = (size_t)TILE_STAGES * 2 * TILE_KEYS * (hd / 8) * sizeof(uint4);
        SPY_ONCE_PER_DEVICE {
            SPY_CUDA(cudaFuncSetAttribute(attention_tiles_kernel<64, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
            SPY_CUDA(cudaFuncSetAttribute(attention_tiles_kernel<128, TW>, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        }
        if (hd == 64) spy_launch(attention_tiles_kernel<64, TW>, grid, dim3(TW * 32), tile_bytes, stream, p);
        else spy_launch(attention_tiles_kernel<128, TW>, grid, dim3(TW * 32), tile_bytes, stream, p);
        SPY_CHECK_LAUNCH("attention_mma (tiles)");
        return 0;
    }
    if (tokens != seqs) SPY_FAIL("attention_mma: split mode needs one token per sequence (%d tokens, %d sequences)", tokens, seqs);
    if (split_keys <= 0 || split_keys % 64 != 0 || max_splits <= 0 || max_splits > 65535)
        SPY_FAIL("attention_mma: split_keys %d must be a positive multiple of 64 and max_splits %d positive", split_keys, max_splits);
    const long long need = spy_attention_mma_scratch_floats(seqs, nh, hd, max_splits);
    if (max_splits > 1 && (scratch == nullptr || scratch_floats < need))
        SPY_FAIL("attention_mma: %lld floats of scratch are needed, %lld were given", need, scratch_floats);
    p.part_o = scratch;
    p.part_ml = scratch ? scratch + (size_t)seqs * nh * max_splits * hd : nullptr;
    if (seqs > 0x7fffffff || nkv > 65535) SPY_FAIL("attention_mma: the batch exceeds the grid limits");
    dim3 grid(seqs, nkv, max_splits);
    const size_t ring_bytes = (size_t)RING * (2 * (hd / 32) + 4 * (hd / 64)) * WARPS * 32 * sizeof(uint4);
    const size_t merge_bytes = (size_t)WARPS * 16 * (hd + 2) * sizeof(float);
    const size_t table_bytes = (size_t)(split_keys + 2) * sizeof(int);   // page_size 1 is the worst case
    const size_t smem = (ring_bytes > merge_bytes ? ring_bytes : merge_bytes) + table_bytes;
    if (smem > 110 * 1024) SPY_FAIL("attention_mma: split_keys %d needs %zu bytes of shared memory (limit %d)", split_keys, smem, 110 * 1024);
    SPY_ONCE_PER_DEVICE {
        SPY_CUDA(cudaFuncSetAttribute(attention_split_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
        SPY_CUDA(cudaFuncSetAttribute(attention_split_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024));
    }
    if (hd == 64) spy_launch(attention_split_kernel<64>, grid, dim3(WARPS * 32), smem, stream, p);
    else spy_launch(attention_split_kernel<128>, grid, dim3(WARPS * 32), smem, stream, p);
    SPY_CHECK_LAUNCH("attention_mma (split)");
    if (max_splits > 1) {
        dim3 mgrid(seqs, nh);
        if (hd == 64) spy_launch(attention_merge_kernel<64>, mgrid, dim3(64), 0, stream, p);
        else spy_launch(attention_merge_kernel<128>, mgrid, dim3(128), 0, stream, p);
        SPY_CHECK_LAUNCH("attention_mma (merge)");
    }
    return 0;
}
