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
// Rotation (optional): pair j of a head, j < rot_half, is rotated by the angle of table entry
// (position, j); the table of (cos, sin) [positions, rot_half] is built in 32-bit by
// spy_build_rope_table; elements from 2*rot_half on pass through.  Which two elements form pair
// j is the pairing rule: 0 ("half") (j, j + rot_half), the reference's (formula:
// src/backends/cpu/cpu_operator.cpp:397-408, table: src/utils/constant_table.hpp:28-41);
// 1 ("interleaved") (2j, 2j + 1), the other rule in use (the reference's doc/op.md:58-95
// describes it, its code does not use it).
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
                                     int page_size, int num_pages, int store, int pairing, int* status)
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
            // pair j = (a, b): a' = a cos - b sin, b' = a sin + b cos
            const bool first = pairing == 0 ? d < rot_half : (d & 1) == 0;
            const int j = pairing == 0 ? (first ? d : d - rot_half) : d >> 1;
            const float2 cs = cos_sin[(size_t)pos * rot_half + j];
            const float lo = buf[pairing == 0 ? j : 2 * j], hi = buf[pairing == 0 ? j + rot_half : 2 * j + 1];
            v = first ? lo * cs.x - hi * cs.y : lo * cs.y + hi * cs.x;
        }
        if (kind == 0) q_dst[d] = from_f32<TQ>(v);
        else dst_page[d] = from_f32<TC>(v);
    }
}

// The common case in one pass over registers: bfloat16 output and cache, head_dim 128, the whole
// head rotated (or no rotation); the input is one bfloat16 array or a stack of float split-K
// partial products, summed in order.  Half a warp owns a (token, head): lane l of it holds
// elements 8l .. 8l + 7 (one 16-byte access of bfloat16); the rotation partner of element
// j < 64 is element j + 64, which lane l ^ 8 holds, so a shuffle replaces the staging in shared
// memory, and the sum of squares is four shuffles.  All loads of an item (input, position,
// block table, rotation table) are issued in rounds without branches before the arithmetic.
template <typename TS, typename TW>
__global__ void __launch_bounds__(256) qk_rope_store_hd128_kernel(const TS* src, int src_splits, long long src_split_stride, bf16* q_out,
                                                                  long long q_out_stride, int tokens, int nh, int nkv,
                                                                  const TW* __restrict__ q_w, const TW* __restrict__ k_w, float eps,
                                                                  const float2* __restrict__ cos_sin, int table_rows,
                                                                  const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                                                  const int* __restrict__ block_table, int table_width, bf16* pages,
                                                                  int page_size, int num_pages, int store, int* status)
{
    constexpr int HD = 128;
    // What depends on no kernel ahead in the stream (the batch's positions and block table, which
    // the host wrote; the rotation table and the norm weights) is loaded before the wait for those
    // kernels; only the input (their product) is read after it.
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, l = lane & 15;
    const int heads = store ? nh + 2 * nkv : nh;
    const int items = tokens * heads;   // the host refuses batches whose items do not fit 31 bits: 32-bit divisions below
    const int mine = (blockIdx.x * (blockDim.x >> 5) + warp) * 2 + (lane >> 4);
    const bool live = mine < items;
    const int item = min(mine, items - 1);   // an item beyond the end repeats the last one and stores nothing
    const int t = item / heads, head = item - t * heads;
    const int kind = head < nh ? 0 : (head < nh + nkv ? 1 : 2);  // q, k, v
    // ---- first loads: the position
    const int pos = positions[t];
    const int seq = kind == 0 ? 0 : seq_of_token[t];
    const TW* w = kind == 0 ? q_w : k_w;
    float wv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) wv[i] = (q_w != nullptr && kind != 2) ? to_f32(w[8 * l + i]) : 1.f;
    // ---- second loads: what the position leads to
    const bool in_table = kind != 0 && pos >= 0 && pos / page_size < table_width;
    const int page = in_table ? block_table[(size_t)seq * table_width + pos / page_size] : -1;
    const bool rotate = kind != 2 && cos_sin != nullptr;
    const bool pos_ok = pos >= 0 && pos < table_rows;
    float4 cs[4];   // (cos, sin) of the pairs 8 (l & 7) .. + 7
    {
        const float4* cs4 = reinterpret_cast<const float4*>(cos_sin + (size_t)((rotate && pos_ok) ? pos : 0) * 64 + 8 * (l & 7));
#pragma unroll
        for (int i = 0; i < 4; ++i) cs[i] = (rotate && pos_ok) ? cs4[i] : make_float4(1.f, 0.f, 1.f, 0.f);
    }
    pdl_wait();
    // ---- the input
    const TS* in = src + (size_t)t * (nh + 2 * nkv) * HD + (size_t)head * HD + 8 * l;
    float v[8];
    if constexpr (sizeof(TS) == 2) {
        const uint4 raw = *reinterpret_cast<const uint4*>(in);
        const uint32_t w4[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w4[i]);
            v[2 * i] = __low2float(a);
            v[2 * i + 1] = __high2float(a);
        }
    } else {
        const float4 f0 = *reinterpret_cast<const float4*>(in), f1 = *reinterpret_cast<const float4*>(in + 4);
        v[0] = f0.x; v[1] = f0.y; v[2] = f0.z; v[3] = f0.w; v[4] = f1.x; v[5] = f1.y; v[6] = f1.z; v[7] = f1.w;
#pragma unroll 4
        for (int s = 1; s < src_splits; ++s) {
            const float4 p0 = *reinterpret_cast<const float4*>(in + (size_t)s * src_split_stride);
            const float4 p1 = *reinterpret_cast<const float4*>(in + (size_t)s * src_split_stride + 4);
            v[0] += p0.x; v[1] += p0.y; v[2] += p0.z; v[3] += p0.w; v[4] += p1.x; v[5] += p1.y; v[6] += p1.z; v[7] += p1.w;
        }
    }
    bf16* dst = nullptr;
    if (live) {
        if (kind == 0) {
            dst = q_out + (size_t)t * q_out_stride + (size_t)head * HD + 8 * l;
        } else if (page < 0 || page >= num_pages) {
            if (l == 0) report_status(status, SPY_STATUS_BAD_PAGE, t);
        } else {
            const int kv_head = kind == 1 ? head - nh : head - nh - nkv;
            dst = pages + ((((size_t)page * 2 + (kind - 1)) * nkv + kv_head) * page_size + pos % page_size) * HD + 8 * l;
        }
        if (rotate && !pos_ok) {
            if (l == 0) report_status(status, SPY_STATUS_BAD_POSITION, t);
            dst = nullptr;
        }
    }
    // ---- norm, rotation, store (both halves of the warp run the shuffles)
    if (q_w != nullptr) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (kind != 2) {
            const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = (inv * v[i]) * wv[i];
        }
    }
    if (cos_sin != nullptr) {
        const float c[8] = {cs[0].x, cs[0].z, cs[1].x, cs[1].z, cs[2].x, cs[2].z, cs[3].x, cs[3].z};
        // lanes 0..7 of the half hold the low half (x_j), lanes 8..15 the high half (x_{j + 64}): the sine enters with its sign
        const float sg = l < 8 ? -1.f : 1.f;
        const float sn[8] = {sg * cs[0].y, sg * cs[0].w, sg * cs[1].y, sg * cs[1].w, sg * cs[2].y, sg * cs[2].w, sg * cs[3].y, sg * cs[3].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float other = __shfl_xor_sync(0xffffffffu, v[i], 8);
            const float r = fmaf(other, sn[i], v[i] * c[i]);   // x_j cos - x_{j+64} sin, or x_j sin + x_{j+64} cos
            if (rotate) v[i] = r;
        }
    }
    if (dst != nullptr) {
        uint4 outv;
        uint32_t* o = reinterpret_cast<uint32_t*>(&outv);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 p = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            o[i] = *reinterpret_cast<uint32_t*>(&p);
        }
        *reinterpret_cast<uint4*>(dst) = outv;
    }
}

// Prompt portions (many tokens, bfloat16 input in one array): half a warp owns FOUR consecutive
// heads of one token (the host takes this kernel only when the heads of a token are a multiple of
// four), so the token's position, page and (cos, sin) row and the two norm weights are loaded once
// for the four, and the four inputs are in flight together.  Lane layout and arithmetic are those
// of the kernel above.
template <typename TW>
__global__ void __launch_bounds__(256, 4) qk_rope_store_hd128_x4_kernel(const bf16* src, bf16* q_out, long long q_out_stride, int tokens, int nh, int nkv,
                                                                     const TW* __restrict__ q_w, const TW* __restrict__ k_w, float eps,
                                                                     const float2* __restrict__ cos_sin, int table_rows,
                                                                     const int* __restrict__ positions, const int* __restrict__ seq_of_token,
                                                                     const int* __restrict__ block_table, int table_width, bf16* pages,
                                                                     int page_size, int num_pages, int store, int* status)
{
    constexpr int HD = 128, PER = 4;
    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, l = lane & 15;
    const int heads = store ? nh + 2 * nkv : nh;
    const int groups = tokens * (heads / PER);   // the host refuses batches whose items do not fit 31 bits
    const int mine = (blockIdx.x * (blockDim.x >> 5) + warp) * 2 + (lane >> 4);
    const bool live = mine < groups;
    const int group = min(mine, groups - 1);   // a group beyond the end repeats the last one and stores nothing
    const int t = group / (heads / PER), head0 = (group - t * (heads / PER)) * PER;
    // ---- what no kernel ahead writes: position, page, rotation row, norm weights
    const int pos = positions[t];
    const int seq = store ? seq_of_token[t] : 0;
    float wq[8], wk[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        wq[i] = q_w != nullptr ? to_f32(q_w[8 * l + i]) : 1.f;
        wk[i] = k_w != nullptr ? to_f32(k_w[8 * l + i]) : 1.f;
    }
    const bool in_table = store && pos >= 0 && pos / page_size < table_width;
    const int page = in_table ? block_table[(size_t)seq * table_width + pos / page_size] : -1;
    const bool pos_ok = pos >= 0 && pos < table_rows;
    const bool have_rot = cos_sin != nullptr;
    float4 cs[4];   // (cos, sin) of the pairs 8 (l & 7) .. + 7
    {
        const float4* cs4 = reinterpret_cast<const float4*>(cos_sin + (size_t)((have_rot && pos_ok) ? pos : 0) * 64 + 8 * (l & 7));
#pragma unroll
        for (int i = 0; i < 4; ++i) cs[i] = (have_rot && pos_ok) ? cs4[i] : make_float4(1.f, 0.f, 1.f, 0.f);
    }
    pdl_wait();
    // ---- the four inputs
    const bf16* in = src + (size_t)t * (nh + 2 * nkv) * HD + (size_t)head0 * HD + 8 * l;
    uint4 raw[PER];
#pragma unroll
    for (int h = 0; h < PER; ++h) raw[h] = *reinterpret_cast<const uint4*>(in + h * HD);
    if (live && have_rot && !pos_ok && l == 0) report_status(status, SPY_STATUS_BAD_POSITION, t);
    const float c[8] = {cs[0].x, cs[0].z, cs[1].x, cs[1].z, cs[2].x, cs[2].z, cs[3].x, cs[3].z};
    // lanes 0..7 of the half hold the low half (x_j), lanes 8..15 the high half (x_{j + 64}): the sine enters with its sign
    const float sg = l < 8 ? -1.f : 1.f;
    const float sn[8] = {sg * cs[0].y, sg * cs[0].w, sg * cs[1].y, sg * cs[1].w, sg * cs[2].y, sg * cs[2].w, sg * cs[3].y, sg * cs[3].w};
#pragma unroll
    for (int h = 0; h < PER; ++h) {
        const int head = head0 + h;
        const int kind = head < nh ? 0 : (head < nh + nkv ? 1 : 2);  // q, k, v
        const uint32_t w4[4] = {raw[h].x, raw[h].y, raw[h].z, raw[h].w};
        float v[8];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&w4[i]);
            v[2 * i] = __low2float(a);
            v[2 * i + 1] = __high2float(a);
        }
        bf16* dst = nullptr;
        if (live && !(have_rot && kind != 2 && !pos_ok)) {
            if (kind == 0) {
                dst = q_out + (size_t)t * q_out_stride + (size_t)head * HD + 8 * l;
            } else if (page < 0 || page >= num_pages) {
                if (l == 0) report_status(status, SPY_STATUS_BAD_PAGE, t);
            } else {
                const int kv_head = kind == 1 ? head - nh : head - nh - nkv;
                dst = pages + ((((size_t)page * 2 + (kind - 1)) * nkv + kv_head) * page_size + pos % page_size) * HD + 8 * l;
            }
        }
        if (q_w != nullptr) {   // both halves of the warp run the shuffles
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (kind != 2) {
                const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] = (inv * v[i]) * (kind == 0 ? wq[i] : wk[i]);
            }
        }
        if (have_rot) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float other = __shfl_xor_sync(0xffffffffu, v[i], 8);
                const float r = fmaf(other, sn[i], v[i] * c[i]);   // x_j cos - x_{j+64} sin, or x_j sin + x_{j+64} cos
                if (kind != 2) v[i] = r;
            }
        }
        if (dst != nullptr) {
            uint4 outv;
            uint32_t* o = reinterpret_cast<uint32_t*>(&outv);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                __nv_bfloat162 pk = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                o[i] = *reinterpret_cast<uint32_t*>(&pk);
            }
            *reinterpret_cast<uint4*>(dst) = outv;
        }
    }
}

template <typename TS, typename TQ, typename TC, typename TW>
static int launch(const void* src, int src_splits, long long src_split_stride, void* q_out, long long q_out_stride, int tokens, int nh, int nkv,
                  int hd, const void* q_w, const void* k_w, float eps, const float* cos_sin, int rot_half, int table_rows, const int* positions,
                  const int* seq_of_token, const int* block_table, int table_width, void* pages, int page_size, int num_pages, int store,
                  int pairing, int* status, cudaStream_t stream)
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
        pairing, status);
    SPY_CHECK_LAUNCH("qk_rope_store");
    return 0;
}

// src: qkv of src_dtype, src_splits arrays src_split_stride elements apart that are summed
// (1 for a plain array).  q_out: [T, ...] rows q_out_stride elements apart, of q_dtype; it may
// be src itself (same dtype, one split, stride (nh + 2 nkv) hd).
// q_w / k_w: null for no norm (both or neither).  cos_sin: null for no rotation.
// store == 0: only the q heads are processed (a layer that reads another layer's cache).
// pairing: 0 pairs (j, j + rot_half), 1 pairs (2j, 2j + 1).
extern "C" int spy_qk_rope_store(const void* src, int src_dtype, int src_splits, long long src_split_stride, void* q_out, int q_dtype,
                                 long long q_out_stride, int tokens, int nh, int nkv, int hd, const void* q_w, const void* k_w, int w_dtype,
                                 float eps, const float* cos_sin, int rot_half, int table_rows, const int* positions, const int* seq_of_token,
                                 const int* block_table, int table_width, void* pages, int cache_dtype, int page_size, int num_pages, int store,
                                 int pairing, int* status, cudaStream_t stream)
{
    if (tokens <= 0) return 0;
    if (pairing != 0 && pairing != 1) SPY_FAIL("qk_rope_store: unknown pairing rule %d (0: halves, 1: interleaved)", pairing);
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
        (cos_sin == nullptr || (rot_half == 64 && pairing == 0)) && q_out_stride % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(q_out) | reinterpret_cast<uintptr_t>(pages)) & 15) == 0) {
        const int heads = store ? nh + 2 * nkv : nh;
        const long long items = (long long)tokens * heads;
        const long long blocks = (items + 15) / 16;   // two items per warp, eight warps per block
        if (items + 16 > 0x7fffffffLL) SPY_FAIL("qk_rope_store: %lld work items exceed the kernel's 31-bit counters", items);
#define SPY_QK_HD128(TS_, splits_, stride_)                                                                                            \
    spy_launch(qk_rope_store_hd128_kernel<TS_, TW>, dim3((int)blocks), dim3(256), 0, stream, (const TS_*)src, splits_, stride_,         \
               (bf16*)q_out, q_out_stride, tokens, nh, nkv, (const TW*)q_w, (const TW*)k_w, eps, (const float2*)cos_sin, table_rows,    \
               positions, seq_of_token, block_table, table_width, (bf16*)pages, page_size, num_pages, store, status)
        if (plain_bf16 && tokens >= 64 && heads % 4 == 0) {
            // prompt portions: four heads of a token per half warp
            const long long groups = items / 4, blocks4 = (groups + 15) / 16;
            SPY_DISPATCH_DTYPE(w_dtype, TW, {
                spy_launch(qk_rope_store_hd128_x4_kernel<TW>, dim3((int)blocks4), dim3(256), 0, stream, (const bf16*)src, (bf16*)q_out, q_out_stride,
                           tokens, nh, nkv, (const TW*)q_w, (const TW*)k_w, eps, (const float2*)cos_sin, table_rows, positions, seq_of_token,
                           block_table, table_width, (bf16*)pages, page_size, num_pages, store, status);
            })
            SPY_CHECK_LAUNCH("qk_rope_store (head_dim 128, four heads a half warp)");
            return 0;
        }
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
                                                  page_size, num_pages, store, pairing, status, stream);
                })
            })
        })
    })
    return 0;
}
