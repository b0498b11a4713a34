// Per-head q/k RMSNorm + rotary position encoding + store of keys and values into the paged
// cache, one kernel over the fused qkv activation.  Replaces five launches of the reference
// (spymaster2h/spyinfer src/models/qwen3.hpp:161-194 and the cache store in
// src/backends/cuda/native/attention.cu:25-47).
//
//   qkv  [T, (nh + 2*nkv) * hd]   q heads, then k heads, then v heads; either one array, or
//        a stack of split-K partial products [splits][T][...] in float that is summed here
//   q    normed and rotated, written to q_out (which may be qkv itself: in place)
//   k    normed and rotated, written to the page of its position (not in place)
//   v    copied to the page of its position
//
// Norm (optional): x * (1/sqrt(mean(x^2) + eps)) * w over head_dim, 32-bit.
// Rotation (optional): pairs (j, j + rot_half) for j < rot_half, angles from a table of
// (cos, sin) [positions, rot_half] built in 32-bit by spy_build_rope_table; elements from
// 2*rot_half on pass through.  Formula: src/backends/cpu/cpu_operator.cpp:397-408,
// table: src/utils/constant_table.hpp:28-41.
//
// Pages of one cache: [num_pages][2 (K, V)][nkv][page_size][hd].  A token at position p of
// sequence s lies in page block_table[s, p / page_size] at slot p % page_size.
#include "common.cuh"

SPY_MODULE(spy_qk_rope_store)

__global__ void rope_table_kernel(float2* __restrict__ table, const float* __restrict__ inv_freq, int rows, int rot_half)
{
    pdl_enter();
    const long long total = (long long)rows * rot_half;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int pos = (int)(i / rot_half), j = (int)(i % rot_half);
        const float angle = (float)pos * inv_freq[j];
        table[i] = make_float2(cosf(angle), sinf(angle));
    }
}

extern "C" int spy_build_rope_table(float* table, const float* inv_freq, int rows, int rot_half, cudaStream_t stream)
{
    if (rows <= 0 || rot_half <= 0) SPY_FAIL("rope table: rows %d and rot_half %d must be positive", rows, rot_half);
    const long long total = (long long)rows * rot_half;
    long long blocks = (total + 255) / 256;
    if (blocks > 4096) blocks = 4096;
    spy_launch(rope_table_kernel, dim3((int)blocks), dim3(256), 0, stream, (float2*)table, inv_freq, rows, rot_half);
    SPY_CHECK_LAUNCH("rope table");
    return 0;
}

constexpr int WARPS_PER_BLOCK = 4;

template <typename TS, typename TQ, typename TC, typename TW>
__global__ void qk_rope_store_kernel(const TS* src, int src_splits, long long src_split_stride, TQ* q_out, long long q_out_stride, int tokens,
                                     int nh, int nkv, int hd, const TW* __restrict__ q_w, const TW* __restrict__ k_w, float eps,
                                     const float2* __restrict__ cos_sin, int rot_half, int table_rows, const int* __restrict__ positions,
                                     const int* __restrict__ seq_of_token, const int* __restrict__ block_table, int table_width, TC* pages,
                                     int page_size, int num_pages, int store, int* status)
{
    extern __shared__ float head_buf[];  // WARPS_PER_BLOCK * hd
    pdl_enter();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = store ? nh + 2 * nkv : nh;
    const long long item = (long long)blockIdx.x * WARPS_PER_BLOCK + warp;
    if (item >= (long long)tokens * heads) return;
    const int t = (int)(item / heads), head = (int)(item % heads);
    const int kind = head < nh ? 0 : (head < nh + nkv ? 1 : 2);  // q, k, v
    float* buf = head_buf + warp * hd;
    const TS* in = src + (size_t)t * (nh + 2 * nkv) * hd + (size_t)head * hd;
    const int pos = positions[t];

    TC* dst_page = nullptr;
    if (kind != 0) {
        const int seq = seq_of_token[t];
        const bool in_table = pos >= 0 && pos / page_size < table_width;
        const int page = in_table ? block_table[(size_t)seq * table_width + pos / page_size] : -1;
        if (page < 0 || page >= num_pages) {
            if (lane == 0) report_status(status, SPY_STATUS_BAD_PAGE, t);
            return;
        }
        const int kv_head = kind == 1 ? head - nh : head - nh - nkv;
        dst_page = pages + ((((size_t)page * 2 + (kind - 1)) * nkv + kv_head) * page_size + pos % page_size) * hd;
    }

    auto read = [&](int d) {
        float v = to_f32(in[d]);
        for (int s = 1; s < src_splits; ++s) v += to_f32(in[(size_t)s * src_split_stride + d]);
        return v;
    };

    if (kind == 2) {
        for (int d = lane; d < hd; d += 32) dst_page[d] = from_f32<TC>(read(d));
        return;
    }

    const TW* w = kind == 0 ? q_w : k_w;
    float ss = 0.f;
    for (int d = lane; d < hd; d += 32) {
        const float v = read(d);
        buf[d] = v;
        ss += v * v;
    }
    if (w != nullptr) {
        ss = warp_sum(ss);
        const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
        for (int d = lane; d < hd; d += 32) buf[d] = (inv * buf[d]) * to_f32(w[d]);
    }
    __syncwarp();
    const bool rotate = cos_sin != nullptr;
    if (rotate && (pos < 0 || pos >= table_rows)) {
        if (lane == 0) report_status(status, SPY_STATUS_BAD_POSITION, t);
        return;
    }
    TQ* q_dst = q_out + (size_t)t * q_out_stride + (size_t)head * hd;
    for (int d = lane; d < hd; d += 32) {
        float v = buf[d];
        if (rotate && d < 2 * rot_half) {
            const int j = d < rot_half ? d : d - rot_half;
            const float2 cs = cos_sin[(size_t)pos * rot_half + j];
            const float lo = buf[j], hi = buf[j + rot_half];
            v = d < rot_half ? lo * cs.x - hi * cs.y : lo * cs.y + hi * cs.x;
        }
        if (kind == 0) q_dst[d] = from_f32<TQ>(v);
        else dst_page[d] = from_f32<TC>(v);
    }
}

// The common case in one pass over registers: bfloat16 everywhere, head_dim 128, the whole head
// rotated (or no rotation), one plain input array.  Lane l of the warp that owns a (token, head)
// holds elements 4l .. 4l + 3 (one 8-byte access); the rotation partner of element j < 64 is
// element j + 64, which lane l ^ 16 holds, so a shuffle replaces the staging in shared memory.
// The input is one bfloat16 array or a stack of float split-K partial products, summed in order.
// A warp takes IPW consecutive (token, head) items (1 as launched) and issues the loads of all of
// them, in rounds without branches, before it works on the first.
template <typename TS, typename TW, int IPW>
__global__ void __launch_bounds__(256) qk_rope_store_hd128_kernel(const TS* src, int src_splits, long long src_split_stride, bf16* q_out,
                                                                  long long q_out_stride, int tokens, int nh, int nkv,
                                                                  const TW* __restrict__ q_w, const TW* __restrict__ k_w, float eps,
                                                                  const float2* __restrict__ cos_sin, int table_rows,
                                                                  const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                                                  const int* __restrict__ block_table, int table_width, bf16* pages,
                                                                  int page_size, int num_pages, int store, int* status)
{
    constexpr int HD = 128;
    pdl_enter();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int heads = store ? nh + 2 * nkv : nh;
    const int items = tokens * heads;   // the host refuses batches whose items do not fit 31 bits: 32-bit divisions below
    const int first = (blockIdx.x * (blockDim.x >> 5) + warp) * IPW;
    if (first >= items) return;
    float v[IPW][4];
    float4 c01[IPW], c23[IPW];
    bf16* dst[IPW];
    int kind[IPW], tok[IPW], pos[IPW], seq[IPW], head_of[IPW];
    // ---- loads of all items, in rounds without branches so that they are in flight together: positions
    // and inputs first, then what a position leads to (block table, rotation table)
#pragma unroll
    for (int k = 0; k < IPW; ++k) {
        const int item = min(first + k, items - 1);   // items beyond the end repeat the last one and store nothing
        tok[k] = item / heads;
        head_of[k] = item - tok[k] * heads;
        kind[k] = head_of[k] < nh ? 0 : (head_of[k] < nh + nkv ? 1 : 2);  // q, k, v
        pos[k] = positions[tok[k]];
        seq[k] = kind[k] == 0 ? 0 : seq_of_token[tok[k]];
        const TS* in = src + (size_t)tok[k] * (nh + 2 * nkv) * HD + (size_t)head_of[k] * HD + 4 * lane;
        if constexpr (sizeof(TS) == 2) {
            const uint2 raw = *reinterpret_cast<const uint2*>(in);
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x), b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
            v[k][0] = __low2float(a); v[k][1] = __high2float(a); v[k][2] = __low2float(b); v[k][3] = __high2float(b);
        } else {
            const float4 f = *reinterpret_cast<const float4*>(in);
            v[k][0] = f.x; v[k][1] = f.y; v[k][2] = f.z; v[k][3] = f.w;
#pragma unroll 8
            for (int s = 1; s < src_splits; ++s) {
                const float4 part = *reinterpret_cast<const float4*>(in + (size_t)s * src_split_stride);
                v[k][0] += part.x; v[k][1] += part.y; v[k][2] += part.z; v[k][3] += part.w;
            }
        }
    }
    int page[IPW];
#pragma unroll
    for (int k = 0; k < IPW; ++k) {
        const bool in_table = kind[k] != 0 && pos[k] >= 0 && pos[k] / page_size < table_width;
        page[k] = in_table ? block_table[(size_t)seq[k] * table_width + pos[k] / page_size] : -1;
        const bool rotate = kind[k] != 2 && cos_sin != nullptr && pos[k] >= 0 && pos[k] < table_rows;
        const float4* cs4 = reinterpret_cast<const float4*>(cos_sin + (size_t)(rotate ? pos[k] : 0) * 64 + 4 * (lane & 15));
        c01[k] = rotate ? cs4[0] : make_float4(1.f, 0.f, 1.f, 0.f);   // (cos, sin) of pairs j, j+1
        c23[k] = rotate ? cs4[1] : make_float4(1.f, 0.f, 1.f, 0.f);   // and of pairs j+2, j+3
    }
#pragma unroll
    for (int k = 0; k < IPW; ++k) {
        dst[k] = nullptr;
        if (first + k >= items) continue;
        if (kind[k] == 0) {
            dst[k] = q_out + (size_t)tok[k] * q_out_stride + (size_t)head_of[k] * HD + 4 * lane;
        } else if (page[k] < 0 || page[k] >= num_pages) {
            if (lane == 0) report_status(status, SPY_STATUS_BAD_PAGE, tok[k]);
        } else {
            const int kv_head = kind[k] == 1 ? head_of[k] - nh : head_of[k] - nh - nkv;
            dst[k] = pages + ((((size_t)page[k] * 2 + (kind[k] - 1)) * nkv + kv_head) * page_size + pos[k] % page_size) * HD + 4 * lane;
        }
        if (kind[k] != 2 && cos_sin != nullptr && (pos[k] < 0 || pos[k] >= table_rows)) {
            if (lane == 0) report_status(status, SPY_STATUS_BAD_POSITION, tok[k]);
            dst[k] = nullptr;
        }
    }
    // ---- norm, rotation, store
#pragma unroll
    for (int k = 0; k < IPW; ++k) {
        if (dst[k] == nullptr) continue;   // uniform over the warp
        const TW* w = kind[k] == 0 ? q_w : k_w;
        if (kind[k] != 2 && w != nullptr) {
            float ss = v[k][0] * v[k][0] + v[k][1] * v[k][1] + v[k][2] * v[k][2] + v[k][3] * v[k][3];
            ss = warp_sum(ss);
            const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[k][i] = (inv * v[k][i]) * to_f32(w[4 * lane + i]);
        }
        if (kind[k] != 2 && cos_sin != nullptr) {
            const float cs_c[4] = {c01[k].x, c01[k].z, c23[k].x, c23[k].z}, cs_s[4] = {c01[k].y, c01[k].w, c23[k].y, c23[k].w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, v[k][i], 16);
                // lanes 0..15 hold the low half (x_j), lanes 16..31 the high half (x_{j + 64})
                v[k][i] = lane < 16 ? v[k][i] * cs_c[i] - other * cs_s[i] : other * cs_s[i] + v[k][i] * cs_c[i];
            }
        }
        __nv_bfloat162 o0 = __floats2bfloat162_rn(v[k][0], v[k][1]), o1 = __floats2bfloat162_rn(v[k][2], v[k][3]);
        uint2 outv;
        outv.x = *reinterpret_cast<uint32_t*>(&o0);
        outv.y = *reinterpret_cast<uint32_t*>(&o1);
        *reinterpret_cast<uint2*>(dst[k]) = outv;
    }
}

template <typename TS, typename TQ, typename TC, typename TW>
static int launch(const void* src, int src_splits, long long src_split_stride, void* q_out, long long q_out_stride, int tokens, int nh, int nkv,
                  int hd, const void* q_w, const void* k_w, float eps, const float* cos_sin, int rot_half, int table_rows, const int* positions,
                  const int* seq_of_token, const int* block_table, int table_width, void* pages, int page_size, int num_pages, int store,
                  int* status, cudaStream_t stream)
{
    const int heads = store ? nh + 2 * nkv : nh;
    const long long items = (long long)tokens * heads;
    const long long blocks = (items + WARPS_PER_BLOCK - 1) / WARPS_PER_BLOCK;
    if (blocks > 0x7fffffffLL) SPY_FAIL("qk_rope_store: %lld work items exceed the grid limit", items);
    const size_t smem = (size_t)WARPS_PER_BLOCK * hd * sizeof(float);
    if (smem > 48 * 1024) SPY_FAIL("qk_rope_store: head_dim %d is too large (limit %d)", hd, 48 * 1024 / 4 / WARPS_PER_BLOCK);
    spy_launch(qk_rope_store_kernel<TS, TQ, TC, TW>, dim3((int)blocks), dim3(WARPS_PER_BLOCK * 32), smem, stream,
        (const TS*)src, src_splits, src_split_stride, (TQ*)q_out, q_out_stride, tokens, nh, nkv, hd, (const TW*)q_w, (const TW*)k_w, eps,
        (const float2*)cos_sin, rot_half, table_rows, positions, seq_of_token, block_table, table_width, (TC*)pages, page_size, num_pages, store,
        status);
    SPY_CHECK_LAUNCH("qk_rope_store");
    return 0;
}

// src: qkv of src_dtype, src_splits arrays src_split_stride elements apart that are summed
// (1 for a plain array).  q_out: [T, ...] rows q_out_stride elements apart, of q_dtype; it may
// be src itself (same dtype, one split, stride (nh + 2 nkv) hd).
// q_w / k_w: null for no norm (both or neither).  cos_sin: null for no rotation.
// store == 0: only the q heads are processed (a layer that reads another layer's cache).
extern "C" int spy_qk_rope_store(const void* src, int src_dtype, int src_splits, long long src_split_stride, void* q_out, int q_dtype,
                                 long long q_out_stride, int tokens, int nh, int nkv, int hd, const void* q_w, const void* k_w, int w_dtype,
                                 float eps, const float* cos_sin, int rot_half, int table_rows, const int* positions, const int* seq_of_token,
                                 const int* block_table, int table_width, void* pages, int cache_dtype, int page_size, int num_pages, int store,
                                 int* status, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || hd <= 0) SPY_FAIL("qk_rope_store: heads %d/%d and head_dim %d must be positive", nh, nkv, hd);
    if (src_splits <= 0) SPY_FAIL("qk_rope_store: src_splits %d must be positive", src_splits);
    if (q_out_stride < (long long)nh * hd) SPY_FAIL("qk_rope_store: q_out rows of %lld elements cannot hold %d heads of %d", q_out_stride, nh, hd);
    if ((q_w == nullptr) != (k_w == nullptr)) SPY_FAIL("qk_rope_store: q and k norm weights must both be given or both be null");
    if (cos_sin && (rot_half <= 0 || 2 * rot_half > hd)) SPY_FAIL("qk_rope_store: rotary width %d does not fit head_dim %d", 2 * rot_half, hd);
    if (store && (page_size <= 0 || num_pages <= 0 || table_width <= 0 || !pages || !block_table))
        SPY_FAIL("qk_rope_store: storing needs pages, a block table and positive page_size/num_pages/table_width");
    const bool plain_bf16 = src_dtype == SPY_BF16 && src_splits == 1;
    const bool float_stack = src_dtype == SPY_F32 && src_split_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0 && q_out != src;
    if ((plain_bf16 || float_stack) && q_dtype == SPY_BF16 && (!store || cache_dtype == SPY_BF16) && hd == 128 &&
        (cos_sin == nullptr || rot_half == 64) && q_out_stride % 4 == 0 &&
        ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(pages)) & 7) == 0) {
        const int heads = store ? nh + 2 * nkv : nh;
        const long long items = (long long)tokens * heads;
        // one item per warp: four per warp with their loads in flight together measured slower
        // (42 against 28 microseconds at 2,048 tokens of 48 heads), the SM holds enough warps as it is
        const long long blocks = (items + 7) / 8;
        if (items + 8 > 0x7fffffffLL) SPY_FAIL("qk_rope_store: %lld work items exceed the kernel's 31-bit counters", items);
#define SPY_QK_HD128(TS_, splits_, stride_)                                                                                            \
    spy_launch(qk_rope_store_hd128_kernel<TS_, TW, 1>, dim3((int)blocks), dim3(256), 0, stream, (const TS_*)src, splits_, stride_,      \
               (bf16*)q_out, q_out_stride, tokens, nh, nkv, (const TW*)q_w, (const TW*)k_w, eps, (const float2*)cos_sin, table_rows,    \
               positions, seq_of_token, block_table, table_width, (bf16*)pages, page_size, num_pages, store, status)
        SPY_DISPATCH_DTYPE(w_dtype, TW, {
            if (plain_bf16) SPY_QK_HD128(bf16, 1, 0LL);
            else SPY_QK_HD128(float, src_splits, src_split_stride);
        })
#undef SPY_QK_HD128
        SPY_CHECK_LAUNCH("qk_rope_store (head_dim 128)");
        return 0;
    }
    SPY_DISPATCH_DTYPE(src_dtype, TS, {
        SPY_DISPATCH_DTYPE(q_dtype, TQ, {
            SPY_DISPATCH_DTYPE(cache_dtype, TC, {
                SPY_DISPATCH_DTYPE(w_dtype, TW, {
                    return launch<TS, TQ, TC, TW>(src, src_splits, src_split_stride, q_out, q_out_stride, tokens, nh, nkv, hd, q_w, k_w, eps,
                                                  cos_sin, rot_half, table_rows, positions, seq_of_token, block_table, table_width, pages,
                                                  page_size, num_pages, store, status, stream);
                })
            })
        })
    })
    return 0;
}
