// bfloat16 attention for decoding (every sequence brings one token) on the 5th-generation
// tensor cores, built to read the paged cache at the speed of the memory.
//
// The products are transposed so that the KEYS fill the 128 rows of the tensor-core tile and the
// G query heads of one key/value head its (padded) 16 columns:
//   S^T = K . Q^T      128 keys x 16 heads, K's tile as it lies in the pages (K-major A operand)
//   softmax            128 threads, ONE KEY PER THREAD: tcgen05.ld brings the key's scores for the G
//                      heads; the running maximum of each head over the tile is one redux per warp
//                      and an exchange of four values through shared memory
//   O^T += V^T . P^T   head_dim x 16 heads; V's tile as it lies in the pages (an MN-major A
//                      operand), P^T written by the softmax threads as bfloat16
// so no tensor-core row is wasted on padding and a tile of 128 keys costs a few hundred cycles
// of one block, far below the time its 64 KB take to arrive.
//
// One persistent block per SM.  The work of the batch is the list of (sequence, kv head, tile of
// 128 keys) units; block c takes units [c * per, (c + 1) * per): a balanced share whatever the
// batch size and the context lengths are.  A block's share is a few SEGMENTS, runs of tiles of
// one (sequence, kv head) pair.  A segment that is a whole pair writes the output; otherwise
// its unnormalised output, maximum and sum go to scratch slot (pair + block), and the warp that
// arrives last at the pair's counter adds the pair's slots in block order and writes the output
// (the counters live in a device array of this library and return to zero with every launch, so
// launches that may overlap on the device must not share it: one stream).
// Roles: warps 0-3 softmax and epilogue; warp 4 allocates tensor memory and issues the MMAs;
// warp 5 brings K tiles, warp 6 V tiles, by TMA boxes of one page x 64 columns straight from
// the paged cache (no cluster multicast), three tiles ahead and across segment borders, so the
// memory pipe stays full from the first tile of a block to its last; warp 7 brings the
// segments' queries.
// Programmatic dependent launch: positions, q_start and the block table are read, and every key
// tile but a pair's last (the one the step's new token lies in) is requested, BEFORE the wait
// for the kernels ahead in the stream, so the cache already streams in while those finish.
// The three arrays must therefore have been written before any kernel that can still be
// running when this one starts (the engine copies them at the start of the step); the queries
// and the new token's page are read after the wait.
// Every wait on an mbarrier is bounded; a wait that runs out raises the block's abort flag,
// which ends all roles, and the status word reports it.
//
// Formula and masking: spymaster2h/spyinfer src/backends/cpu/cpu_attention.cpp:89-135; this
// replaces its paged_attention_decode_kernel (src/backends/cuda/native/attention.cu:257-370),
// which reads the cache once per query head on the CUDA cores.
// Limits (checked on the host): head_dim 64 or 128, G <= 16, bfloat16, a page size of 8, 16, 32,
// 64 or 128 tokens, at most 1024 sequences.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

SPY_MODULE(spy_attention_decode)

namespace {

using namespace tc;

constexpr int TILE = 128;            // keys per tile = UMMA M of the first product
constexpr int NCOLS = 16;            // UMMA N: the heads of one key/value head, padded
constexpr int STAGES = 3;            // K and V tiles in flight
constexpr int QSLOTS = 4;            // queries of segments in flight
constexpr int MAX_SEQS = 1024;
constexpr int NUM_THREADS = 256;
constexpr int MAX_PAIRS = 65536;     // (sequence, kv head) pairs of one launch
constexpr int HALF_BYTES = TILE * 128;        // 128 rows of 64 elements
constexpr int STAGE_BYTES = 2 * HALF_BYTES;   // a K or V tile: two halves of head_dim
constexpr int QP_BYTES = 2 * NCOLS * 128;     // Q^T or P^T: 16 rows, two halves of 64 elements
constexpr float LOG2E = 1.4426950408889634f;
constexpr float RESCALE_THRESHOLD = 8.0f;

constexpr int K_OFF = 0;
constexpr int V_OFF = K_OFF + STAGES * STAGE_BYTES;
constexpr int Q_OFF = V_OFF + STAGES * STAGE_BYTES;
constexpr int P_OFF = Q_OFF + QSLOTS * QP_BYTES;
constexpr int PREFIX_OFF = P_OFF + 2 * QP_BYTES;                 // int[MAX_SEQS + 1]
constexpr int POS_OFF = PREFIX_OFF + (MAX_SEQS + 4) * 4;         // int[MAX_SEQS]: every sequence's position (-1: skipped)
constexpr int RED_OFF = POS_OFF + MAX_SEQS * 4;                  // float[2][4][16] maxima, float[4][16] sums
constexpr int BAR_OFF = RED_OFF + (2 * 4 * NCOLS + 4 * NCOLS) * 4;
constexpr int NUM_BARS = 4 * STAGES + 3 * 2 + 2 * QSLOTS + 2 + 1;
constexpr int SMEM_TOTAL = BAR_OFF + NUM_BARS * 8 + 32 + 1024;   // then slack to align the base to 1024
constexpr int TMEM_COLS = 64;                                    // S^T: 2 x 16 columns; O^T: 16 columns from 32

struct Params {
    bf16* out;                 // [T, nh * hd]
    const int* block_table;    // [S, table_width]
    const int* positions;      // [T]
    const int* q_start;        // [S + 1]
    float* part_o;             // [slots][G][HD] unnormalised partial outputs
    float* part_ml;            // [slots][G][2]  (maximum in the log2 domain, sum)
    int* status;
    int table_width, page_size, num_pages, nh, nkv, G, S, window, blocks, max_keys, mode;
    int hd;                    // the head size as stored (a multiple of 8, at most HD): the tiles are HD wide, what lies beyond hd is zero
    float scale_log2;
};

// A block's share of the batch's units: either the contiguous range [u0, u1) of the list of all
// (sequence, kv head, tile) units, which cuts pairs wherever the range ends, or (whole) the pairs
// first, first + stride, ... each with all its tiles.
struct Share {
    const int* prefix;   // [S + 1] tiles of the sequences before s
    int S, nkv, u0, u1, first, stride;
    bool whole;
};

// A run of tiles [t, t_end) of pair (s, kvh), whose keys span `tiles` tiles; `left` units (or, whole,
// the next pair's index) remain for the block after this run.
struct Seg {
    int s, kvh, t0, t, t_end, tiles, left;
};

__device__ __forceinline__ bool seg_whole(Seg& g, const Share& sh, int pair)
{
    for (; pair < sh.S * sh.nkv; pair += sh.stride) {
        g.s = pair / sh.nkv;
        g.tiles = sh.prefix[g.s + 1] - sh.prefix[g.s];
        if (g.tiles == 0) continue;
        g.kvh = pair - g.s * sh.nkv;
        g.t0 = g.t = 0;
        g.t_end = g.tiles;
        g.left = pair + sh.stride;
        return true;
    }
    return false;
}

__device__ __forceinline__ bool seg_first(Seg& g, const Share& sh)
{
    if (sh.whole) return seg_whole(g, sh, sh.first);
    if (sh.u0 >= sh.u1) return false;
    int a = 0, b = sh.S;   // nkv * prefix[a] <= u0 < nkv * prefix[b]
    while (b - a > 1) {
        const int mid = (a + b) >> 1;
        if (sh.nkv * sh.prefix[mid] <= sh.u0) a = mid; else b = mid;
    }
    g.s = a;
    g.tiles = sh.prefix[a + 1] - sh.prefix[a];
    const int r = sh.u0 - sh.nkv * sh.prefix[a];
    g.kvh = r / g.tiles;
    g.t0 = g.t = r - g.kvh * g.tiles;
    const int n = min(g.tiles - g.t, sh.u1 - sh.u0);
    g.t_end = g.t + n;
    g.left = sh.u1 - sh.u0 - n;
    return true;
}

__device__ __forceinline__ bool seg_next(Seg& g, const Share& sh)
{
    if (sh.whole) return seg_whole(g, sh, g.left);
    if (g.left <= 0) return false;
    if (++g.kvh == sh.nkv) {
        g.kvh = 0;
        do {
            if (++g.s >= sh.S) return false;
            g.tiles = sh.prefix[g.s + 1] - sh.prefix[g.s];
        } while (g.tiles == 0);
    }
    const int n = min(g.tiles, g.left);
    g.t0 = g.t = 0;
    g.t_end = n;
    g.left -= n;
    return true;
}

// the keys a sequence's token sees: [lo, pos]; tiles of 128 keys at absolute positions
__device__ __forceinline__ void key_range(const Params& p, const int* pos_s, int s, int& pos, int& lo)
{
    pos = pos_s[s];
    lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
}

__device__ __forceinline__ int tiles_of(int pos, int lo) { return pos >= 0 ? pos / TILE - lo / TILE + 1 : 0; }


// arrivals of the warps that hold a part of a pair's result; the last one merges and resets it
__device__ int g_pair_arrivals[MAX_PAIRS];

// floats map to integers of the same order (and back: the map is its own inverse)
__device__ __forceinline__ int ordered(float f)
{
    const int i = __float_as_int(f);
    return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float unordered(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }

template <int HD, int GN>
__global__ void __maxnreg__(160)
attention_decode_kernel(const __grid_constant__ CUtensorMap page_map, const __grid_constant__ CUtensorMap q_map, const Params p)
{
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    int* prefix = reinterpret_cast<int*>(smem + PREFIX_OFF);
    int* pos_s = reinterpret_cast<int*>(smem + POS_OFF);
    float* red = reinterpret_cast<float*>(smem + RED_OFF);            // [2][4][NCOLS]
    float* lred = red + 2 * 4 * NCOLS;                                // [4][NCOLS]
    uint64_t* bar_kfull = reinterpret_cast<uint64_t*>(smem + BAR_OFF);   // [STAGES] K tile landed (TMA bytes)
    uint64_t* bar_kfree = bar_kfull + STAGES;                            // [STAGES] its product is complete (MMA commit)
    uint64_t* bar_vfull = bar_kfree + STAGES;
    uint64_t* bar_vfree = bar_vfull + STAGES;
    uint64_t* bar_s = bar_vfree + STAGES;                                // [2] scores complete (MMA commit)
    uint64_t* bar_p = bar_s + 2;                                         // [2] probabilities written (128 arrivals)
    uint64_t* bar_o = bar_p + 2;                                         // [2] V^T.P^T complete (MMA commit)
    uint64_t* bar_qfull = bar_o + 2;                                     // [QSLOTS] a segment's queries landed
    uint64_t* bar_qfree = bar_qfull + QSLOTS;                            // [QSLOTS] the segment's first products are complete
    uint64_t* bar_red = bar_qfree + QSLOTS;                              // [2] the four warps' maxima are written
    uint64_t* bar_lred = bar_red + 2;                                    // the four warps' sums are written
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_lred + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* s_max_tiles = reinterpret_cast<int*>(tmem_slot + 2);   // the most tiles any sequence has

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, tid = threadIdx.x;
    if (tid == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&page_map) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&q_map) : "memory");
        for (int i = 0; i < STAGES; ++i) {
            mbar_init(bar_kfull + i, 1);
            mbar_init(bar_kfree + i, 1);
            mbar_init(bar_vfull + i, 1);
            mbar_init(bar_vfree + i, 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(bar_s + i, 1);
            mbar_init(bar_p + i, TILE);
            mbar_init(bar_o + i, 1);
            mbar_init(bar_red + i, 4);
        }
        for (int i = 0; i < QSLOTS; ++i) {
            mbar_init(bar_qfull + i, 1);
            mbar_init(bar_qfree + i, 1);
        }
        mbar_init(bar_lred, 4);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 4) tmem_alloc(tmem_slot, TMEM_COLS);
    // rows of Q^T beyond the G heads are never copied: keep them zero (their columns of S^T and O^T are not used)
    for (int i = tid; i < QSLOTS * QP_BYTES / 16; i += NUM_THREADS) reinterpret_cast<uint4*>(smem + Q_OFF)[i] = make_uint4(0, 0, 0, 0);
    fence_async_proxy();

    // ---- the batch's units: tiles of every sequence, prefix sums, this block's share
    for (int s = tid; s < p.S; s += NUM_THREADS) {
        const int tok = p.q_start[s];
        int pos = p.positions[tok];
        if (pos < 0 || pos >= p.max_keys) {   // outside the block table: the sequence is skipped and reported
            pos = -1;
            if (blockIdx.x == 0) report_status(p.status, SPY_STATUS_BAD_POSITION, tok);
        }
        pos_s[s] = pos;
        prefix[s + 1] = tiles_of(pos, p.window > 0 ? max(0, pos - p.window + 1) : 0);
    }
    __syncthreads();
    if (warp == 0) {
        int carry = 0, most = 0;
        for (int base = 0; base < p.S; base += 32) {
            const int s = base + lane;
            int v = s < p.S ? prefix[s + 1] : 0;
            most = max(most, v);
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int up = __shfl_up_sync(0xffffffffu, v, o);
                if (lane >= o) v += up;
            }
            if (s < p.S) prefix[s + 1] = carry + v;
            carry += __shfl_sync(0xffffffffu, v, 31);
        }
        most = __reduce_max_sync(0xffffffffu, most);
        if (lane == 0) {
            prefix[0] = 0;
            *s_max_tiles = most;
        }
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_o = tmem_base + 2 * NCOLS;
    const int units = p.nkv * prefix[p.S];
    const int per = (units + (int)gridDim.x - 1) / (int)gridDim.x;
    const int u0 = min(units, (int)blockIdx.x * per), u1 = min(units, u0 + per);
    // Whole pairs, dealt round-robin, need no merge; they pay when the blocks then end about when an
    // even split of the units would (short contexts, or many pairs per block).
    const int pairs = p.S * p.nkv, rounds = (pairs + (int)gridDim.x - 1) / (int)gridDim.x;
    // (measured at 1 to 200 requests of 640 to 8,192 keys: a tile costs about 1.05 us in the busiest block, the merges of an even
    // split about four tiles' time, a little more with many pairs: whole pairs while rounds x longest <= 1.125 x share + 4)
    const bool whole = p.mode == 2 || (p.mode == 0 && (long long)rounds * *s_max_tiles * 8 <= (long long)per * 9 + 32);
    const Share share = {prefix, p.S, p.nkv, u0, u1, (int)blockIdx.x, (int)gridDim.x, whole};
    const uint32_t k_s = smem_u32(smem + K_OFF), v_s = smem_u32(smem + V_OFF), q_s = smem_u32(smem + Q_OFF), p_s = smem_u32(smem + P_OFF);

    if (warp < 4) {
        // ---------------------------------------------------------------- softmax (one key per thread) and epilogue
        const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
        Seg g;
        bool more = seg_first(g, share), alive = true;
        int gt = 0, seg = 0;   // tiles and segments this block has begun
        while (more && alive) {
            int pos, lo;
            key_range(p, pos_s, g.s, pos, lo);
            const int tok = p.q_start[g.s];
            const int tile_first = lo / TILE;
            float m_used[GN], l[GN];   // the maximum the probabilities are taken against (equal in all threads); this thread's share of the sum
#pragma unroll
            for (int n = 0; n < GN; ++n) {
                m_used[n] = -INFINITY;
                l[n] = 0.f;
            }
            for (; g.t < g.t_end; ++g.t, ++gt) {
                const int st = gt & 1;
                const uint32_t ph = (uint32_t)(gt >> 1) & 1;
                if (!(alive = mbar_wait(bar_s + st, ph, abort_flag))) break;
                fence_after_sync();
                uint32_t r[GN];
                tmem_load<GN>(tmem_base + st * NCOLS + lane_addr, r);
                tmem_wait_ld();
                const int j = (tile_first + g.t) * TILE + tid;
                const bool visible = j >= lo && j <= pos;
                float sc[GN];
#pragma unroll
                for (int n = 0; n < GN; ++n) {
                    sc[n] = visible ? __uint_as_float(r[n]) * p.scale_log2 : -INFINITY;
                    const int mx = __reduce_max_sync(0xffffffffu, ordered(sc[n]));
                    if (lane == n) red[(st * 4 + warp) * NCOLS + n] = unordered(mx);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_red + st);
                if (!(alive = mbar_wait(bar_red + st, ph, abort_flag))) break;
                // the maximum in use moves only when a head's maximum grew by more than the threshold (or from nothing)
                float alpha[GN];
                bool grew = false;
#pragma unroll
                for (int n = 0; n < GN; ++n) {
                    const float* rr = red + st * 4 * NCOLS + n;
                    const float m_new = fmaxf(fmaxf(m_used[n], fmaxf(rr[0], rr[NCOLS])), fmaxf(rr[2 * NCOLS], rr[3 * NCOLS]));
                    const bool grow = m_new > m_used[n] + RESCALE_THRESHOLD || (m_used[n] == -INFINITY && m_new != -INFINITY);
                    alpha[n] = grow ? (m_used[n] == -INFINITY ? 0.f : fast_exp2(m_used[n] - m_new)) : 1.f;
                    if (grow) {
                        l[n] *= alpha[n];
                        m_used[n] = m_new;
                        grew = true;
                    }
                }
                uint16_t pb[GN];
#pragma unroll
                for (int n = 0; n < GN; ++n) {
                    const float pr = fast_exp2(sc[n] - (m_used[n] == -INFINITY ? 0.f : m_used[n]));
                    l[n] += pr;
                    pb[n] = __bfloat16_as_ushort(__float2bfloat16_rn(pr));
                }
                // O^T is rescaled once the product of the tile before is complete (the segment's first product overwrites it)
                if (grew && g.t > g.t0) {
                    if (!(alive = mbar_wait(bar_o + ((gt - 1) & 1), (uint32_t)((gt - 1) >> 1) & 1, abort_flag))) break;
                    fence_after_sync();
                    uint32_t o[GN];
                    tmem_load<GN>(tmem_o + lane_addr, o);
                    tmem_wait_ld();
#pragma unroll
                    for (int n = 0; n < GN; ++n) o[n] = __float_as_uint(__uint_as_float(o[n]) * alpha[n]);
                    tmem_store<GN>(tmem_o + lane_addr, o);
                    tmem_wait_st();
                }
                // P^T's stage is free when the product of two tiles back is complete
                if (gt >= 2 && !(alive = mbar_wait(bar_o + st, (uint32_t)((gt - 2) >> 1) & 1, abort_flag))) break;
                uint8_t* pdst = smem + P_OFF + st * QP_BYTES + (tid >> 6) * (NCOLS * 128) + (tid & 7) * 2;
                const int chunk = (tid & 63) >> 3;
#pragma unroll
                for (int n = 0; n < GN; ++n) *reinterpret_cast<uint16_t*>(pdst + n * 128 + ((chunk ^ (n & 7)) << 4)) = pb[n];
                fence_async_proxy();
                fence_before_sync();
                mbar_arrive(bar_p + st);
            }
            if (!alive) break;
            // ---- the segment's result: O^T / sum, or the partial result of this run of tiles
            if (!(alive = mbar_wait(bar_o + ((gt - 1) & 1), (uint32_t)((gt - 1) >> 1) & 1, abort_flag))) break;
            fence_after_sync();
            uint32_t o[GN];
            tmem_load<GN>(tmem_o + lane_addr, o);
            tmem_wait_ld();
#pragma unroll
            for (int n = 0; n < GN; ++n) {
                const float v = warp_sum(l[n]);
                if (lane == n) lred[warp * NCOLS + n] = v;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_lred);
            if (!(alive = mbar_wait(bar_lred, (uint32_t)seg & 1, abort_flag))) break;
            const bool direct = g.t0 == 0 && g.t_end == g.tiles;
            const int pair = g.s * p.nkv + g.kvh;
            const size_t slot = (size_t)pair + blockIdx.x;
            float sums[GN];
#pragma unroll
            for (int n = 0; n < GN; ++n) sums[n] = (lred[n] + lred[NCOLS + n]) + (lred[2 * NCOLS + n] + lred[3 * NCOLS + n]);
            if (direct) {
#pragma unroll
                for (int n = 0; n < GN; ++n)
                    if (n < p.G && tid < p.hd)
                        p.out[((size_t)tok * p.nh + g.kvh * p.G + n) * p.hd + tid] = __float2bfloat16_rn(sums[n] > 0.f ? __uint_as_float(o[n]) / sums[n] : 0.f);
            } else {
#pragma unroll
                for (int n = 0; n < GN; ++n) {
                    if (n >= p.G) break;
                    if (tid < HD) p.part_o[(slot * p.G + n) * HD + tid] = __uint_as_float(o[n]);
                    if (tid == n) {
                        p.part_ml[(slot * p.G + n) * 2] = m_used[n];
                        p.part_ml[(slot * p.G + n) * 2 + 1] = sums[n];
                    }
                }
                // the pair's blocks: every warp of each arrives once; the last warp to arrive merges
                const int off = p.nkv * prefix[g.s] + g.kvh * g.tiles;
                const int c_first = off / per, c_last = (off + g.tiles - 1) / per;
                __threadfence();
                __syncwarp();
                int last = 0;
                if (lane == 0) {
                    last = atomicAdd(&g_pair_arrivals[pair], 1) == 4 * (c_last - c_first + 1) - 1;
                    if (last) g_pair_arrivals[pair] = 0;
                }
                last = __shfl_sync(0xffffffffu, last, 0);
                if (last) {
                    // 32 / GN lanes share a head; a lane merges W consecutive columns of its head.  The
                    // loads of CH parts are issued together (a pair of two to four parts then costs one
                    // round trip to L2 instead of one per part); the parts are added in block order and
                    // the running maximum rescales what has been added so far.
                    __threadfence();
                    constexpr int LPH = 32 / GN, W = HD / LPH, CH = W <= 16 ? 4 : (W <= 32 ? 2 : 1);
                    const int n = lane / LPH, col = (lane % LPH) * W;
                    if (n < p.G) {
                        const float* ml0 = p.part_ml + ((size_t)pair * p.G + n) * 2;
                        const float* o0 = p.part_o + ((size_t)pair * p.G + n) * HD + col;
                        float M = -INFINITY, L = 0.f, acc[W];
#pragma unroll
                        for (int i = 0; i < W; ++i) acc[i] = 0.f;
                        for (int c0 = c_first; c0 <= c_last; c0 += CH) {
                            float2 ml[CH];
                            float4 part[CH][W / 4];
#pragma unroll
                            for (int j = 0; j < CH; ++j) {
                                const size_t sl = (size_t)min(c0 + j, c_last) * p.G;   // beyond the last: the last again, counted for nothing
                                ml[j] = __ldcg(reinterpret_cast<const float2*>(ml0 + sl * 2));
#pragma unroll
                                for (int i = 0; i < W / 4; ++i) part[j][i] = __ldcg(reinterpret_cast<const float4*>(o0 + sl * HD) + i);
                            }
#pragma unroll
                            for (int j = 0; j < CH; ++j) {
                                const float mj = c0 + j <= c_last ? ml[j].x : -INFINITY;
                                const float m_new = fmaxf(M, mj);
                                const float keep = M == -INFINITY ? 0.f : exp2f(M - m_new);
                                const float f = mj == -INFINITY ? 0.f : exp2f(mj - m_new);
                                M = m_new;
                                L = L * keep + ml[j].y * f;
#pragma unroll
                                for (int i = 0; i < W / 4; ++i) {
                                    acc[4 * i] = acc[4 * i] * keep + part[j][i].x * f;
                                    acc[4 * i + 1] = acc[4 * i + 1] * keep + part[j][i].y * f;
                                    acc[4 * i + 2] = acc[4 * i + 2] * keep + part[j][i].z * f;
                                    acc[4 * i + 3] = acc[4 * i + 3] * keep + part[j][i].w * f;
                                }
                            }
                        }
                        bf16* dst = p.out + ((size_t)tok * p.nh + g.kvh * p.G + n) * p.hd + col;
                        const float inv = L > 0.f ? 1.f / L : 0.f;
#pragma unroll
                        for (int i = 0; i < W; i += 8) {
                            uint4 v;
                            uint32_t* u = reinterpret_cast<uint32_t*>(&v);
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const __nv_bfloat162 t2 = __floats2bfloat162_rn(acc[i + 2 * e] * inv, acc[i + 2 * e + 1] * inv);
                                u[e] = *reinterpret_cast<const uint32_t*>(&t2);
                            }
                            if (col + i < p.hd) *reinterpret_cast<uint4*>(dst + i) = v;
                        }
                    }
                }
            }
            ++seg;
            more = seg_next(g, share);
        }
    } else if (warp == 4) {
        // ---------------------------------------------------------------- MMA issue
        if (lane == 0) {
            const uint32_t idesc_qk = instr_desc_bf16(TILE, NCOLS, false, false), idesc_pv = instr_desc_bf16(TILE, NCOLS, true, false);
            Seg gq, gp;
            bool moreq = seg_first(gq, share), morep = seg_first(gp, share), ok = true;
            int iq = 0, segq = 0;
            auto issue_qk = [&]() {   // S^T of the next tile
                const int stage = iq % STAGES, slot = segq % QSLOTS;
                if (gq.t == gq.t0) ok = mbar_wait(bar_qfull + slot, (uint32_t)(segq / QSLOTS) & 1, abort_flag);
                ok = ok && mbar_wait(bar_kfull + stage, (uint32_t)(iq / STAGES) & 1, abort_flag);
                if (!ok) return;
                fence_after_sync();
                const uint32_t kb = k_s + stage * STAGE_BYTES, qb = q_s + slot * QP_BYTES;
#pragma unroll
                for (int s = 0; s < HD / 16; ++s)   // 16 elements of head_dim: 32 bytes along the rows of a 64-element half
                    umma(tmem_base + (iq & 1) * NCOLS, desc_k_major(kb + (s >> 2) * HALF_BYTES + (s & 3) * 32),
                         desc_k_major(qb + (s >> 2) * (NCOLS * 128) + (s & 3) * 32), idesc_qk, s > 0 ? 1u : 0u);
                umma_commit(bar_s + (iq & 1));
                umma_commit(bar_kfree + stage);
                ++iq;
                if (++gq.t == gq.t_end) {
                    umma_commit(bar_qfree + slot);
                    ++segq;
                    moreq = seg_next(gq, share);
                }
            };
            if (moreq) issue_qk();
            if (ok && moreq) issue_qk();
            for (int ip = 0; morep && ok; ++ip) {
                const int st = ip & 1, stage = ip % STAGES;
                ok = mbar_wait(bar_p + st, (uint32_t)(ip >> 1) & 1, abort_flag) && mbar_wait(bar_vfull + stage, (uint32_t)(ip / STAGES) & 1, abort_flag);
                if (!ok) break;
                fence_after_sync();
                const uint32_t vb = v_s + stage * STAGE_BYTES, pb = p_s + st * QP_BYTES;
#pragma unroll
                for (int s = 0; s < TILE / 16; ++s)   // 16 keys: 16 rows of V, 32 bytes along the rows of P^T
                    umma(tmem_o, desc_mn_major(vb + s * 16 * 128, HALF_BYTES), desc_k_major(pb + (s >> 2) * (NCOLS * 128) + (s & 3) * 32), idesc_pv,
                         (gp.t > gp.t0 || s > 0) ? 1u : 0u);
                umma_commit(bar_o + st);
                umma_commit(bar_vfree + stage);
                if (++gp.t == gp.t_end) morep = seg_next(gp, share);
                if (moreq) issue_qk();   // S^T's stage st is free: P^T of this tile was made from it
            }
        }
    } else if (warp == 7) {
        // ---------------------------------------------------------------- TMA: the segments' queries, which the kernel ahead wrote
        if (lane == 0) {
            Seg g;
            bool more = seg_first(g, share);
            int tok_next = more ? p.q_start[g.s] : 0;   // the host wrote q_start: read ahead of the wait and of each segment's load
            pdl_wait();
            for (int seg = 0; more; ++seg) {
                const int slot = seg % QSLOTS;
                const int tok = tok_next;
                if (seg >= QSLOTS && !mbar_wait(bar_qfree + slot, (uint32_t)(seg / QSLOTS - 1) & 1, abort_flag)) break;
                mbar_expect_tx(bar_qfull + slot, (uint32_t)p.G * HD * 2);
#pragma unroll
                for (int h = 0; h < HD / 64; ++h)
                    tma_load_3d(q_s + slot * QP_BYTES + h * (NCOLS * 128), &q_map, h * 64, g.kvh * p.G, tok, bar_qfull + slot);
                more = seg_next(g, share);
                if (more) tok_next = p.q_start[g.s];
            }
        }
    } else {
        // ---------------------------------------------------------------- TMA: K tiles (warp 5), V tiles (warp 6)
        // One box per page and 64-column half, one lane each (a single thread issuing them one after
        // the other is the slower way: small boxes are bound by issue latency, not by bandwidth).
        const int kv = warp - 5;
        uint64_t* bar_full = kv == 0 ? bar_kfull : bar_vfull;
        uint64_t* bar_free = kv == 0 ? bar_kfree : bar_vfree;
        const uint32_t ring = kv == 0 ? k_s : v_s;
        const int pages_per_tile = TILE / p.page_size;
        const int boxes = pages_per_tile * (HD / 64);                        // at most 32
        const uint32_t box_bytes = (uint32_t)p.page_size * 128;              // page_size rows of 64 elements
        const int my_page = lane / (HD / 64), my_half = lane % (HD / 64);
        Seg g;
        bool more = seg_first(g, share), ok = true, waited = false;
        int i = 0;
        while (more && ok) {
            int pos, lo;
            key_range(p, pos_s, g.s, pos, lo);
            const int tile_first = lo / TILE;
            const int* bt = p.block_table + (size_t)g.s * p.table_width;
            for (; g.t < g.t_end; ++g.t, ++i) {
                const int stage = i % STAGES;
                if (!waited && g.t == g.tiles - 1) {   // the pair's last tile holds the token the kernel ahead has just stored
                    pdl_wait();
                    waited = true;
                }
                // This lane's page of the tile (read before the wait for the stage, which hides the lookup).
                // Every box of the tile is copied, so that no row of the stage is ever stale: pages that hold
                // none of the sequence's keys, or that the table does not name, are replaced by page 0, whose
                // rows are finite like any page's and meet probabilities of zero.
                const int lp = (tile_first + g.t) * pages_per_tile + my_page;
                const bool in_range = lp * p.page_size <= pos && (lp + 1) * p.page_size > lo;
                int page = (lane < boxes && in_range && lp < p.table_width) ? bt[lp] : 0;
                if (lane == 0 && lp + 4 * pages_per_tile < p.table_width) asm volatile("prefetch.global.L2 [%0];" ::"l"(bt + lp + 4 * pages_per_tile));
                if (page < 0 || page >= p.num_pages) {
                    if (kv == 0) report_status(p.status, SPY_STATUS_BAD_PAGE, p.q_start[g.s]);
                    page = 0;
                }
                if (lane == 0) {
                    if (i >= STAGES) ok = mbar_wait(bar_free + stage, (uint32_t)(i / STAGES - 1) & 1, abort_flag);
                    if (ok) mbar_expect_tx(bar_full + stage, (uint32_t)boxes * box_bytes);
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                if (!ok) break;
                if (lane < boxes) {
                    const int y = ((page * 2 + kv) * p.nkv + g.kvh) * p.page_size;
                    tma_load_2d(ring + stage * STAGE_BYTES + my_half * HALF_BYTES + my_page * p.page_size * 128, &page_map, my_half * 64, y, bar_full + stage);
                }
            }
            if (ok) more = seg_next(g, share);
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
    if (warp == 4) {
        fence_after_sync();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

int sm_count() { return spy_sm_count(); }

template <int HD, int GN>
int launch(const CUtensorMap& page_map, const CUtensorMap& q_map, const Params& p, cudaStream_t stream)
{
    SPY_ONCE_PER_DEVICE {
        SPY_CUDA(cudaFuncSetAttribute(attention_decode_kernel<HD, GN>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL));
    }
    spy_launch(attention_decode_kernel<HD, GN>, dim3(p.blocks), dim3(NUM_THREADS), (size_t)SMEM_TOTAL, stream, page_map, q_map, p);
    SPY_CHECK_LAUNCH("attention_decode");
    return 0;
}

}  // namespace


// Floats of scratch a batch of `seqs` decoding sequences needs: one slot per (sequence, kv head) pair and per block.
extern "C" long long spy_attention_decode_scratch_floats(int seqs, int nh, int nkv, int hd)
{
    if (nkv <= 0 || nh % nkv != 0) return 0;
    return ((long long)seqs * nkv + sm_count()) * (nh / nkv) * ((hd <= 64 ? 64 : 128) + 2);
}

// Attention of a decoding batch over its pages: every sequence brings one token (row
// q_start[s] of q, at positions[q_start[s]]).  mode 0: the kernel decides how the work is shared
// out; 1: the units split evenly, pairs cut where a block's share ends; 2: whole pairs.
extern "C" int spy_attention_decode(const void* q, long long q_row_stride, void* out, const void* pages, const int* block_table, int table_width,
                                    int page_size, int num_pages, int nh, int nkv, int hd, const int* positions, const int* q_start, int tokens,
                                    int seqs, int window, float scale, int mode, float* scratch, long long scratch_floats, int* status,
                                    cudaStream_t stream)
{
    if (tokens <= 0 || seqs <= 0) return 0;
    if (nh <= 0 || nkv <= 0 || nh % nkv != 0) SPY_FAIL("attention_decode: %d query heads do not group over %d key/value heads", nh, nkv);
    const int G = nh / nkv;
    if (G > NCOLS) SPY_FAIL("attention_decode: %d query heads per key/value head exceed %d", G, NCOLS);
    if (hd < 8 || hd > 128 || hd % 8 != 0) SPY_FAIL("attention_decode: head_dim %d is not a multiple of 8 between 8 and 128", hd);
    const int hd_tile = hd <= 64 ? 64 : 128;   // the kernel's tile width: the TMA boxes fill what lies beyond hd with zeros
    if (seqs > MAX_SEQS || (long long)seqs * nkv > MAX_PAIRS)
        SPY_FAIL("attention_decode: %d sequences of %d key/value heads exceed %d sequences or %d pairs", seqs, nkv, MAX_SEQS, MAX_PAIRS);
    if (q_row_stride % 8 != 0 || q_row_stride < (long long)nh * hd || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(pages) & 15))
        SPY_FAIL("attention_decode: queries and pages must be 16-byte aligned with rows a multiple of 8 elements");
    if (num_pages <= 0 || table_width <= 0) SPY_FAIL("attention_decode: num_pages and table_width must be positive");
    if (page_size < 8 || page_size > TILE || TILE % page_size != 0)
        SPY_FAIL("attention_decode: page_size %d must be 8, 16, 32, 64 or 128 (one TMA box per page)", page_size);
    if (window < 0) SPY_FAIL("attention_decode: window %d must be 0 (none) or positive", window);
    if (mode < 0 || mode > 2) SPY_FAIL("attention_decode: mode %d is not 0 (the kernel decides), 1 (units split evenly) or 2 (whole pairs)", mode);
    const long long max_keys = (long long)table_width * page_size;
    if (max_keys >= (1LL << 30) || (long long)seqs * nkv * (max_keys / TILE + 1) >= (1LL << 31))
        SPY_FAIL("attention_decode: %d sequences of up to %lld keys exceed this kernel's counters", seqs, max_keys);
    const int sms = sm_count();
    if (sms <= 0) SPY_FAIL("attention_decode: the device's SM count is not available");
    const long long need = spy_attention_decode_scratch_floats(seqs, nh, nkv, hd);
    if (scratch == nullptr || scratch_floats < need) SPY_FAIL("attention_decode: %lld floats of scratch are needed, %lld were given", need, scratch_floats);
    tc::EncodeTiledFn encode = tc::encode_tiled_fn();
    if (encode == nullptr) SPY_FAIL("attention_decode: cuTensorMapEncodeTiled is not available from the driver");

    Params p;
    p.out = (bf16*)out; p.block_table = block_table; p.positions = positions; p.q_start = q_start; p.status = status;
    p.part_o = scratch; p.part_ml = scratch + ((size_t)seqs * nkv + sms) * G * hd_tile;
    p.table_width = table_width; p.page_size = page_size; p.num_pages = num_pages; p.nh = nh; p.nkv = nkv; p.G = G; p.S = seqs;
    p.window = window; p.hd = hd; p.blocks = sms; p.max_keys = (int)max_keys; p.mode = mode; p.scale_log2 = scale * LOG2E;

    // the pages of this cache as one matrix [num_pages * 2 * nkv * page_size rows, hd]; a box is one page's rows x 64 columns
    CUtensorMap page_map, q_map;
    {
        cuuint64_t dims[2] = {(cuuint64_t)hd, (cuuint64_t)num_pages * 2 * nkv * page_size};
        cuuint64_t strides[1] = {(cuuint64_t)hd * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)page_size};
        cuuint32_t elem[2] = {1, 1};
        CUresult r = encode(&page_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pages), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) SPY_FAIL("attention_decode: cuTensorMapEncodeTiled (pages) failed with code %d", (int)r);
    }
    {   // the queries as [tokens][nh heads][hd]; a box is the G heads of one kv head x 64 columns of one token
        cuuint64_t dims[3] = {(cuuint64_t)hd, (cuuint64_t)nh, (cuuint64_t)tokens};
        cuuint64_t strides[2] = {(cuuint64_t)hd * 2, (cuuint64_t)q_row_stride * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, 1};
        cuuint32_t elem[3] = {1, 1, 1};
        CUresult r = encode(&q_map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) SPY_FAIL("attention_decode: cuTensorMapEncodeTiled (queries) failed with code %d", (int)r);
    }
    const int gn = G <= 4 ? 4 : (G <= 8 ? 8 : 16);
    if (hd_tile == 64) return gn == 4 ? launch<64, 4>(page_map, q_map, p, stream) : (gn == 8 ? launch<64, 8>(page_map, q_map, p, stream) : launch<64, 16>(page_map, q_map, p, stream));
    return gn == 4 ? launch<128, 4>(page_map, q_map, p, stream) : (gn == 8 ? launch<128, 8>(page_map, q_map, p, stream) : launch<128, 16>(page_map, q_map, p, stream));
}
