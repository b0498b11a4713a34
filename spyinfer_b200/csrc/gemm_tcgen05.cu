// bfloat16 matrix product on the 5th-generation tensor cores:  C[M, N] = A[M, K] . W[N, K]^T
// with 32-bit accumulation in tensor memory.  Both operands are K-major; TMA brings
// 128-byte-swizzled tiles into a ring of shared-memory stages, one elected thread issues
// tcgen05.mma (128 x BN x 16 per instruction), four warps read the accumulator back with
// tcgen05.ld and store bfloat16 or float32.
//
// Three kernels, chosen by the number of tokens M:
//   up to 256 tokens (gemm_tcgen05_kernel): one block computes one tile over a range of K with the
//     weights in the instruction's M slot (up to 128 outputs) and a tile of 16, 32 or 64 tokens in
//     its N slot; the tile is stored transposed.  With split-K every split stores its 32-bit
//     partial tile into scratch memory and the consumer (or a second kernel) sums the splits in a
//     fixed order; the number of splits depends only on the shape class, so a token's result
//     does not depend on the batch beyond rounding;
//   more tokens (gemm_tcgen05_persistent_kernel): 128 tokens x 256 outputs a tile, one block an SM;
//   512 tokens and more (gemm_tcgen05_pair_kernel): 256 x 256 tiles on pairs of blocks.
// Tails: rows beyond M or N and the end of K are zero-filled by TMA; stores are predicated.
// K must be a multiple of 8 (16-byte rows for TMA).  No cluster multicast is used.
//
// The reference's products are cuBLAS half-precision GEMMs and a SIMT GEMV
// (spymaster2h/spyinfer src/backends/cuda/cublas/sgemm.cu:37-55,
// src/backends/cuda/native/sgemm.cu:130-206); it has no tensor-core kernel of its own.
#include <cuda.h>

#include "common.cuh"
#include "tcgen05.cuh"

SPY_MODULE(spy_gemm_tcgen05)

namespace {

using namespace tc;

constexpr int BM = 128;            // rows of X per tile = UMMA M
constexpr int BK = 64;             // 64 bf16 = 128 bytes = one swizzle row
constexpr int UMMA_K = 16;
constexpr int NUM_THREADS = 192;   // warp 0: TMA, warp 1: MMA + TMEM, warps 2..5: epilogue

// The one-tile kernel (few tokens): BN tokens in the N slot, up to 128 weight rows in the M slot.
// Two blocks share an SM, each with AREA bytes of stages.  The stages are packed: a tile of fewer
// than 128 weight rows takes only its own bytes (rounded up to the swizzle's 1 KB), so more stages
// fit the area and as many bytes stay in flight as with full tiles.  The tensor core still reads
// 128 rows: the spare ones come from whatever lies behind (the next stage; the area ends with
// room for that) and feed accumulator rows that are never stored.
template <int BN> struct Tile {
    static constexpr int X_BYTES = BM * BK * 2;
    static constexpr int Y_BYTES = BN * BK * 2;
    static constexpr int TMEM_COLS = BN < 32 ? 32 : BN;
    static constexpr int AREA = 110 * 1024;
    static constexpr int MAX_STAGES = 12;
    static constexpr size_t SMEM = (size_t)AREA + 1024 /* alignment slack */ + 256 /* barriers */;
    __host__ __device__ static constexpr int x_bytes(int tile_rows) { return (tile_rows * BK * 2 + 1023) & ~1023; }
    __host__ __device__ static constexpr int stages(int tile_rows)
    {
        const int n = (AREA - (X_BYTES - x_bytes(tile_rows))) / (x_bytes(tile_rows) + Y_BYTES);
        return n < MAX_STAGES ? n : MAX_STAGES;
    }
};

// The persistent kernel on single blocks (many tokens): 128 tokens x 256 weight rows a tile, one block an SM.
struct WideTile {
    static constexpr int BN = 256;
    static constexpr int X_BYTES = BM * BK * 2;
    static constexpr int Y_BYTES = BN * BK * 2;
    static constexpr int STAGE_BYTES = X_BYTES + Y_BYTES;
    static constexpr int STAGES = (200 * 1024) / STAGE_BYTES;
    static constexpr size_t SMEM = (size_t)STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
};

template <typename TC> __device__ __forceinline__ void store_elem(TC* p, float v) { *p = from_f32<TC>(v); }

// Stores 32 consecutive columns of one row, vectorised when the row allows it.
template <typename TC>
__device__ __forceinline__ void store_row32(TC* dst, const uint32_t (&r)[32], int valid, bool aligned)
{
    if (valid >= 32 && aligned) {
        if constexpr (sizeof(TC) == 4) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(dst)[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]),
                                                                __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                uint4 v;
                __nv_bfloat162 t;
                t = __floats2bfloat162_rn(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1])); v.x = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3])); v.y = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5])); v.z = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(__uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7])); v.w = *reinterpret_cast<uint32_t*>(&t);
                reinterpret_cast<uint4*>(dst)[i] = v;
            }
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < valid) store_elem(dst + i, __uint_as_float(r[i]));
    }
}

__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }   // the four epilogue warps
constexpr int PLAIN_STAGE_LD = 132;   // floats between the tokens of a staged plain tile (128 weight rows and a pad, rows 16 bytes aligned)
constexpr int SWIGLU_STAGE_LD = 66;   // bf16 elements between the tokens of a staged SwiGLU tile (64 outputs and a pad)

// silu(g) * u for a bfloat16 result: the fast exponential and division (2 ulp of float each) are far
// inside the result's rounding, and the accurate ones cost the epilogue warps more instructions than all
// the rest of a tile's read-out (64 tokens: 4.0 against 1.5 microseconds).  A gate below -87 gives
// g / inf = -0, the limit.  The 32-bit path has its own SwiGLU kernel with the accurate functions.
__device__ __forceinline__ float silu_mul(float g, float u) { return __fdividef(g, 1.0f + __expf(-g)) * u; }

// X: the weights [x_rows, K] in the instruction's M slot; Y: the tokens [y_rows, K] in its N slot;
// out[y, x] (row stride ld).  splits > 1: out is the float scratch [splits][rows][ld] and TC is float.
// EPI == 1 (SwiGLU): the weight's rows alternate gate, up, gate, up, ...; the kernel stores
// silu(gate) * up, half as many output columns (ld counts those); one pass over K only.
template <int BN, typename TC, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 2)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, TC* __restrict__ out,
                    long long ld, long long split_stride, int x_rows, int y_rows, int k_blocks, int k_blocks_per_split, int tile_rows,
                    int* status, const uint8_t* __restrict__ next_weights, long long next_bytes)
{
    using T = Tile<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + T::AREA);
    uint64_t* empty_bar = full_bar + T::MAX_STAGES;
    uint64_t* accum_bar = empty_bar + T::MAX_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accum_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // tile_rows (<= BM) rows of X belong to this block: the box of map_x has that many rows, the rest of
    // the stage's 128 rows is stale and feeds accumulator rows that are never stored
    // the token tile is the grid's fastest dimension, so that the blocks that share a weight tile
    // (65 to 256 tokens are two to four tiles of 64) start together and the later ones find it in L2
    const int x0 = blockIdx.y * tile_rows, y0 = blockIdx.x * BN;
    const uint32_t stage_tx = (uint32_t)tile_rows * BK * 2 + T::Y_BYTES;
    const int x_bytes = T::x_bytes(tile_rows), stage_bytes = x_bytes + T::Y_BYTES, stages = T::stages(tile_rows);
    const int kb0 = blockIdx.z * k_blocks_per_split;
    const int kb1 = min(k_blocks, kb0 + k_blocks_per_split);
    const int num_kb = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((uint32_t)T::TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    pdl_launch_dependents();   // the next kernel in the stream may begin its own prologue
    if (warp == 0) {
        if (lane == 0) {
            // The weight operand (X when swapped, Y otherwise) depends on no earlier kernel: its
            // tiles for the first stages are requested before the wait for the kernels ahead in
            // the stream, so weights already stream in while those are finishing.
            const int pre = min(num_kb, stages);
            for (int i = 0; i < pre; ++i) {
                uint8_t* xs = tiles + (size_t)i * stage_bytes;
                mbar_expect_tx(full_bar + i, stage_tx);
                tma_load_2d(smem_u32(xs), &map_x, (kb0 + i) * BK, x0, full_bar + i);
            }
            pdl_wait();
            for (int i = 0; i < pre; ++i) {
                uint8_t* xs = tiles + (size_t)i * stage_bytes;
                tma_load_2d(smem_u32(xs + x_bytes), &map_y, (kb0 + i) * BK, y0, full_bar + i);
            }
            int s = 0;
            uint32_t phase = 1;   // of the round before: the first wait on a stage is for its first release
            for (int i = pre; i < num_kb; ++i) {
                if (!mbar_wait(empty_bar + s, phase ^ 1, abort_flag)) break;
                uint8_t* xs = tiles + (size_t)s * stage_bytes;
                uint8_t* ys = xs + x_bytes;
                mbar_expect_tx(full_bar + s, stage_tx);
                tma_load_2d(smem_u32(xs), &map_x, (kb0 + i) * BK, x0, full_bar + s);
                tma_load_2d(smem_u32(ys), &map_y, (kb0 + i) * BK, y0, full_bar + s);
                if (++s == stages) {
                    s = 0;
                    phase ^= 1;
                }
            }
            // Every load of this block has been requested.  What follows this product in a decode step is a
            // stretch of short kernels (a norm, the q/k rotation, the attention's start) that move few bytes
            // and leave the memory idle, and then a product whose weights are known now: this block asks for
            // its share of them to be brought into L2 meanwhile.  A hint only: nothing waits for it.
            if (next_bytes > 0) {
                const long long blocks = (long long)gridDim.x * gridDim.y * gridDim.z;
                const long long me = blockIdx.x + (long long)gridDim.x * (blockIdx.y + (long long)gridDim.y * blockIdx.z);
                const long long share = ((next_bytes + blocks - 1) / blocks + 127) / 128 * 128;
                long long at = me * share;
                const long long end = at + share < next_bytes ? at + share : next_bytes;
                for (; at < end; at += 16384) {
                    const long long n = end - at < 16384 ? end - at : 16384;
                    l2_prefetch(next_weights + at, (uint32_t)(n & ~15LL));
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc_bf16(BM, BN, false, false);
            int s = 0;
            uint32_t phase = 0;
            for (int i = 0; i < num_kb; ++i) {
                if (!mbar_wait(full_bar + s, phase, abort_flag)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint8_t* xs = tiles + (size_t)s * stage_bytes;
                const uint64_t dx = desc_k_major(smem_u32(xs)), dy = desc_k_major(smem_u32(xs + x_bytes));
#pragma unroll
                for (int k = 0; k < BK / UMMA_K; ++k) {
                    const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);
                    umma(tmem_base, dx + adv, dy + adv, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                umma_commit(empty_bar + s);   // the stage is free again when these MMAs have read it
                if (++s == stages) {
                    s = 0;
                    phase ^= 1;
                }
            }
            umma_commit(accum_bar);           // the accumulator is complete when every MMA has finished
        }
    } else {
        // epilogue: warp w reads TMEM lanes 32*(w%4) .. +31, i.e. tile rows of X
        const int quarter = warp & 3;
        pdl_wait();   // the output buffer may still be in use by a kernel ahead in the stream
        const bool ok = mbar_wait(accum_bar, 0, abort_flag);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int x = quarter * 32 + lane < tile_rows ? x0 + quarter * 32 + lane : x_rows;   // rows beyond the tile's are the next block's
        TC* base = out + (size_t)blockIdx.z * split_stride;
        if (ok && num_kb > 0) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c;
                if constexpr (BN >= 32) tmem_load<32>(taddr, r);
                else tmem_load<16>(taddr, *reinterpret_cast<uint32_t(*)[16]>(&r[0]));
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                const int cols = BN >= 32 ? 32 : BN;
                const int y = y0 + c;
                if constexpr (EPI == 1) {
                    // lanes 2i and 2i + 1 hold gate row and up row of output x / 2 for every token.  Two tokens
                    // at a time: the even lane sends the second token's gate and finishes the first token, the
                    // odd lane sends the first token's up and finishes the second, so every lane computes.
                    // The results go to shared memory (the stages are free by now) and from there to the
                    // output in rows: a 2-byte store per token and lane straight from here queues behind the
                    // weight tiles that the next product's blocks on this SM have already asked for.
                    const bool odd = (lane & 1) != 0;
                    bf16* staged = reinterpret_cast<bf16*>(tiles);
#pragma unroll
                    for (int j = 0; j < 32; j += 2) {
                        if (j < cols) {
                            const float a = __uint_as_float(r[j]), b = __uint_as_float(r[j + 1]);
                            const float got = __shfl_xor_sync(0xffffffffu, odd ? a : b, 1);
                            const float v = silu_mul(odd ? got : a, odd ? b : got);
                            staged[(c + j + (odd ? 1 : 0)) * SWIGLU_STAGE_LD + ((quarter * 32 + lane) >> 1)] = __float2bfloat16_rn(v);
                        }
                    }
                } else if constexpr (BN >= 32) {
                    // 32 tokens and more: through shared memory as well, so that the output leaves in rows of
                    // 16 bytes a lane (a quarter of the store requests of 4 bytes a lane and token)
                    float* staged = reinterpret_cast<float*>(tiles);
#pragma unroll
                    for (int j = 0; j < 32; ++j) staged[(c + j) * PLAIN_STAGE_LD + quarter * 32 + lane] = __uint_as_float(r[j]);
                } else {
                    if (x < x_rows) {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (j < cols && y + j < y_rows) store_elem(base + (size_t)(y + j) * ld + x, __uint_as_float(r[j]));
                    }
                }
            }
            if constexpr (EPI == 0 && BN >= 32) {
                epilogue_barrier();
                const float* staged = reinterpret_cast<const float*>(tiles);
                const int e = quarter * 32 + lane;
                const int outs = min(tile_rows, x_rows - x0), rows = min(BN, y_rows - y0);
                TC* gout = base + (size_t)y0 * ld + x0;
                if ((outs & 3) == 0 && (ld & 3) == 0 && (reinterpret_cast<uintptr_t>(gout) & 15) == 0) {
                    const int quads = outs >> 2;
                    for (int i = e; i < rows * quads; i += 128) {
                        const int t = i / quads, q = i - t * quads;
                        const float4 v = *reinterpret_cast<const float4*>(staged + t * PLAIN_STAGE_LD + 4 * q);
                        TC* dst = gout + (size_t)t * ld + 4 * q;
                        if constexpr (sizeof(TC) == 4) {
                            *reinterpret_cast<float4*>(dst) = v;
                        } else {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                            uint2 w;
                            w.x = *reinterpret_cast<uint32_t*>(&lo);
                            w.y = *reinterpret_cast<uint32_t*>(&hi);
                            *reinterpret_cast<uint2*>(dst) = w;
                        }
                    }
                } else {
                    for (int i = e; i < rows * outs; i += 128) {
                        const int t = i / outs, q = i - t * outs;
                        store_elem(gout + (size_t)t * ld + q, staged[t * PLAIN_STAGE_LD + q]);
                    }
                }
            }
            if constexpr (EPI == 1) {
                // rows of the staged tile to the output, 4 bytes a lane where the row allows it
                epilogue_barrier();
                const bf16* staged = reinterpret_cast<const bf16*>(tiles);
                const int e = quarter * 32 + lane;
                const int outs = min(tile_rows, x_rows - x0) / 2, rows = min(BN, y_rows - y0);
                TC* gout = base + (size_t)y0 * ld + x0 / 2;
                if ((outs & 1) == 0 && (ld & 1) == 0 && (reinterpret_cast<uintptr_t>(gout) & 3) == 0) {
                    const int words = outs / 2;
                    for (int i = e; i < rows * words; i += 128) {
                        const int t = i / words, q = i - t * words;
                        *reinterpret_cast<uint32_t*>(gout + (size_t)t * ld + 2 * q) = *reinterpret_cast<const uint32_t*>(staged + t * SWIGLU_STAGE_LD + 2 * q);
                    }
                } else {
                    for (int i = e; i < rows * outs; i += 128) {
                        const int t = i / outs, q = i - t * outs;
                        gout[(size_t)t * ld + q] = staged[t * SWIGLU_STAGE_LD + q];
                    }
                }
            }
        } else if (num_kb <= 0) {
            // an empty K range contributes zeros (only possible for a trailing split)
            for (int c = 0; c < BN; ++c) {
                const int y = y0 + c;
                if (x < x_rows && y < y_rows) {
                    store_elem(base + (size_t)y * ld + x, 0.f);
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        // a wait ran out: give copies that may still be in flight time to land before the
        // shared memory is released, then report
        if (threadIdx.x == 0) {
            const unsigned long long t0 = global_timer();
            while (global_timer() - t0 < 2000000ull) { }
            report_status(status, SPY_STATUS_WAIT_TIMEOUT, (int)(blockIdx.x + blockIdx.y * gridDim.x));
        }
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)T::TMEM_COLS) : "memory");
    }
}

// Stores 32 consecutive accumulator columns of row x (normal mode), with the optional SwiGLU.
template <typename TC, int EPI>
__device__ __forceinline__ void store_chunk_normal(TC* base, long long ld, int x, int y, int x_rows, int y_rows, const uint32_t (&r)[32])
{
    if (x >= x_rows || y >= y_rows) return;
    if constexpr (EPI == 1) {
        uint32_t o[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(silu_mul(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1])));
        TC* dst = base + (size_t)x * ld + y / 2;
        const int valid = min(16, (y_rows - y) / 2);
        if (valid >= 16 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0 && sizeof(TC) == 2) {
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                uint4 v;
                __nv_bfloat162 t;
                t = __floats2bfloat162_rn(__uint_as_float(o[8 * i]), __uint_as_float(o[8 * i + 1])); v.x = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 2]), __uint_as_float(o[8 * i + 3])); v.y = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 4]), __uint_as_float(o[8 * i + 5])); v.z = *reinterpret_cast<uint32_t*>(&t);
                t = __floats2bfloat162_rn(__uint_as_float(o[8 * i + 6]), __uint_as_float(o[8 * i + 7])); v.w = *reinterpret_cast<uint32_t*>(&t);
                reinterpret_cast<uint4*>(dst)[i] = v;
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j)
                if (j < valid) store_elem(dst + j, __uint_as_float(o[j]));
        }
    } else {
        TC* dst = base + (size_t)x * ld + y;
        const bool aligned = (reinterpret_cast<uintptr_t>(dst) & 15) == 0;
        store_row32<TC>(dst, r, min(32, y_rows - y), aligned);
    }
}

// The product for many tokens (normal mode, 128 x 256 tiles, one pass over K) as a PERSISTENT
// kernel: one block per SM walks tiles blockIdx.x, blockIdx.x + gridDim.x, ...; the TMA ring
// runs on across tiles, and the accumulator is double-buffered in tensor memory (2 x 256
// columns), so the epilogue of a tile (tcgen05.ld, conversion, stores) overlaps the main loop
// of the next.  Tiles are numbered with the token tiles fastest, so blocks that run side by
// side share a weight tile in L2.
// How the persistent kernel deals out its work.  stream_tiles == 0: whole tiles, block b takes
// tiles b, b + blocks, ...  Otherwise (stream-K) the first stream_tiles tiles are shared out by
// K blocks: their K blocks are numbered through, tile after tile, and block b takes the numbers
// [b * per_block, (b + 1) * per_block); the tiles behind them are taken whole as before.  Every SM
// then gets the same share of the product, where whole tiles would leave SMs idle.  The host shares
// the tiles out only when there are fewer tiles than SMs (a few hundred tokens): with more, whole
// tiles round by round are faster although the last round is not full, because the blocks of a
// round walk K in step and the tiles of a row or column block meet in L2.
// A block's share is cut into segments, each a range of K blocks of one tile.  A segment that
// holds a tile's first K block OWNS the tile: if it ends before the tile does (it is then the
// last segment of the block's share), the following blocks hold the rest (each as its FIRST
// segment, long finished by then), leave their 32-bit partial tiles in the workspace and raise a
// flag; the owner adds them in block order and stores the tile.  Flags return to zero by themselves.
struct Segment {
    int tile, kb0, kb1;
};
struct SegmentWalk {
    long long at, end;    // K-block numbers of this block's share of the stream tiles
    int tile, num_tiles;  // the block's next whole tile
    int k_blocks;
    __device__ SegmentWalk(int num_tiles_, int k_blocks_, int stream_tiles, int per_block) : num_tiles(num_tiles_), k_blocks(k_blocks_)
    {
        const long long total = (long long)stream_tiles * k_blocks;
        at = (long long)blockIdx.x * per_block;
        end = at + per_block < total ? at + per_block : total;
        tile = stream_tiles + blockIdx.x;
    }
    __device__ bool next(Segment& s)
    {
        if (at < end) {
            s.tile = (int)(at / k_blocks);
            s.kb0 = (int)(at - (long long)s.tile * k_blocks);
            const long long left = end - at;
            s.kb1 = left < k_blocks - s.kb0 ? s.kb0 + (int)left : k_blocks;
            at += s.kb1 - s.kb0;
            return true;
        }
        if (tile < num_tiles) {
            s.tile = tile;
            s.kb0 = 0;
            s.kb1 = k_blocks;
            tile += gridDim.x;
            return true;
        }
        return false;
    }
};
// a partial tile in the workspace: [32-column chunk][quad of the chunk][row][4 floats], so that a
// warp's 16-byte accesses are contiguous
__device__ __forceinline__ size_t partial_index(int c, int j, int row) { return ((size_t)((c >> 5) * 8 + j) * BM + row) * 4; }
constexpr int STREAM_MAX_BLOCKS = 1024;
constexpr int STREAM_MIN_KB = 8;   // a block's share is at least this many K blocks
constexpr int STREAM_TILE_FLOATS = BM * 256;
__device__ int g_stream_flags[STREAM_MAX_BLOCKS];

template <typename TC, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_persistent_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, TC* __restrict__ out,
                               long long ld, int x_rows, int y_rows, int k_blocks, int x_tiles, int num_tiles, int stream_tiles, int per_block,
                               float* workspace, int* status)
{
    using T = WideTile;
    constexpr int BN = T::BN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)T::STAGES * T::STAGE_BYTES);
    uint64_t* empty_bar = full_bar + T::STAGES;
    uint64_t* acc_full = empty_bar + T::STAGES;    // [2] accumulator complete (MMA commit)
    uint64_t* acc_empty = acc_full + 2;            // [2] accumulator read out (128 arrivals)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < T::STAGES; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full + b, 1);
            mbar_init(acc_empty + b, 128);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(2u * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    pdl_launch_dependents();
    if (warp == 0) {
        if (lane == 0) {
            long long g = 0;   // k-blocks requested so far: the ring position
            bool first = true, ok = true;
            SegmentWalk walk(num_tiles, k_blocks, stream_tiles, per_block);
            Segment sg;
            while (ok && walk.next(sg)) {
                const int x0 = (sg.tile % x_tiles) * BM, y0 = (sg.tile / x_tiles) * BN;
                int kb = sg.kb0;
                if (first) {
                    // weights (Y) of the first stages before the wait for the kernels ahead in the stream
                    const int pre = min(sg.kb1 - sg.kb0, T::STAGES);
                    for (int i = 0; i < pre; ++i) {
                        mbar_expect_tx(full_bar + i, T::STAGE_BYTES);
                        tma_load_2d(smem_u32(tiles + (size_t)i * T::STAGE_BYTES + T::X_BYTES), &map_y, (sg.kb0 + i) * BK, y0, full_bar + i);
                    }
                    pdl_wait();
                    for (int i = 0; i < pre; ++i) tma_load_2d(smem_u32(tiles + (size_t)i * T::STAGE_BYTES), &map_x, (sg.kb0 + i) * BK, x0, full_bar + i);
                    kb = sg.kb0 + pre;
                    g = pre;
                    first = false;
                }
                for (; kb < sg.kb1; ++kb, ++g) {
                    const int s = (int)(g % T::STAGES);
                    const uint32_t phase = (uint32_t)(g / T::STAGES) & 1;
                    if (g >= T::STAGES && !mbar_wait(empty_bar + s, phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* xs = tiles + (size_t)s * T::STAGE_BYTES;
                    mbar_expect_tx(full_bar + s, T::STAGE_BYTES);
                    tma_load_2d(smem_u32(xs), &map_x, kb * BK, x0, full_bar + s);
                    tma_load_2d(smem_u32(xs + T::X_BYTES), &map_y, kb * BK, y0, full_bar + s);
                }
            }
            if (first) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = instr_desc_bf16(BM, BN, false, false);
            long long g = 0;
            int i = 0;
            bool ok = true;
            SegmentWalk walk(num_tiles, k_blocks, stream_tiles, per_block);
            Segment sg;
            for (; ok && walk.next(sg); ++i) {
                const int buf = i & 1;
                const uint32_t aph = (uint32_t)(i >> 1) & 1;
                if (i >= 2) ok = mbar_wait(acc_empty + buf, aph ^ 1, abort_flag);   // the epilogue has read this buffer's last tile
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t acc = tmem_base + (uint32_t)buf * BN;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++g) {
                    const int s = (int)(g % T::STAGES);
                    const uint32_t phase = (uint32_t)(g / T::STAGES) & 1;
                    ok = mbar_wait(full_bar + s, phase, abort_flag);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint8_t* xs = tiles + (size_t)s * T::STAGE_BYTES;
                    const uint64_t dx = desc_k_major(smem_u32(xs)), dy = desc_k_major(smem_u32(xs + T::X_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);
                        umma(acc, dx + adv, dy + adv, idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit(empty_bar + s);
                }
                if (ok) umma_commit(acc_full + buf);
            }
        }
    } else {
        const int quarter = warp & 3;
        pdl_wait();   // the output buffer may still be in use by a kernel ahead in the stream
        int i = 0;
        bool ok = true;
        SegmentWalk walk(num_tiles, k_blocks, stream_tiles, per_block);
        Segment sg;
        for (; ok && walk.next(sg); ++i) {
            const int buf = i & 1;
            const uint32_t aph = (uint32_t)(i >> 1) & 1;
            const int x0 = (sg.tile % x_tiles) * BM, y0 = (sg.tile / x_tiles) * BN;
            ok = mbar_wait(acc_full + buf, aph, abort_flag);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int row = quarter * 32 + lane, x = x0 + row;
            if (sg.kb0 > 0) {
                // the rest of a tile that a block before this one owns: the partial tile goes to the workspace
                float* mine = workspace + (size_t)blockIdx.x * STREAM_TILE_FLOATS;
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_load<32>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        __stcg(reinterpret_cast<float4*>(mine + partial_index(c, j, row)),
                               make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                mbar_arrive(acc_empty + buf);
                __threadfence();
                epilogue_barrier();
                if (row == 0) {
                    __threadfence();
                    atomicExch(&g_stream_flags[blockIdx.x], 1);
                }
                continue;
            }
            const int helpers_kb = k_blocks - sg.kb1;   // K blocks of this tile that the following blocks hold
            int helper = blockIdx.x + 1;
            if (helpers_kb > 0) {
                // every following block holds per_block K blocks of the rest, the last one what is left
                for (int rest = helpers_kb, h = helper; rest > 0 && ok; rest -= per_block, ++h) {
                    const unsigned long long t0 = global_timer();
                    while (atomicAdd(&g_stream_flags[h], 0) == 0) {
                        if (global_timer() - t0 > WAIT_LIMIT_NS) {
                            *abort_flag = 1;
                            ok = false;
                            break;
                        }
                    }
                }
                __threadfence();
            }
            if (helpers_kb > 0 && ok) {
                // the helpers' partial chunks are requested two chunks ahead of their use: a round trip to L2
                // a chunk would otherwise hold the accumulator, and with it the tensor core, for microseconds
                float4 pre[3][8];
                auto fetch = [&](int c, float4 (&dst)[8]) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) dst[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                    for (int rest = helpers_kb, h = helper; rest > 0; rest -= per_block, ++h) {
                        const float* theirs = workspace + (size_t)h * STREAM_TILE_FLOATS;
                        float4 v[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) v[j] = __ldcg(reinterpret_cast<const float4*>(theirs + partial_index(c, j, row)));
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            dst[j].x += v[j].x;
                            dst[j].y += v[j].y;
                            dst[j].z += v[j].z;
                            dst[j].w += v[j].w;
                        }
                    }
                };
                fetch(0, pre[0]);
                fetch(32, pre[1]);
#pragma unroll
                for (int ci = 0; ci < BN / 32; ++ci) {
                    const int c = ci * 32;
                    if (ci + 2 < BN / 32) fetch(c + 64, pre[(ci + 2) % 3]);
                    uint32_t r[32];
                    tmem_load<32>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 v = pre[ci % 3][j];
                        r[4 * j] = __float_as_uint(__uint_as_float(r[4 * j]) + v.x);
                        r[4 * j + 1] = __float_as_uint(__uint_as_float(r[4 * j + 1]) + v.y);
                        r[4 * j + 2] = __float_as_uint(__uint_as_float(r[4 * j + 2]) + v.z);
                        r[4 * j + 3] = __float_as_uint(__uint_as_float(r[4 * j + 3]) + v.w);
                    }
                    store_chunk_normal<TC, EPI>(out, ld, x, y0 + c, x_rows, y_rows, r);
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_load<32>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c), r);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    store_chunk_normal<TC, EPI>(out, ld, x, y0 + c, x_rows, y_rows, r);
                }
            }
            if (helpers_kb > 0) {
                // every thread has read the partial tiles: their flags go back to zero for the next product
                epilogue_barrier();
                if (row == 0)
                    for (int rest = helpers_kb, h = helper; rest > 0; rest -= per_block, ++h) g_stream_flags[h] = 0;
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(acc_empty + buf);
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            const unsigned long long t0 = global_timer();
            while (global_timer() - t0 < 2000000ull) { }
            report_status(status, SPY_STATUS_WAIT_TIMEOUT, (int)blockIdx.x);
        }
        __syncthreads();
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2u * BN) : "memory");
    }
}

// The product for many tokens on PAIRS of blocks (cta_group::2): a cluster of two blocks on
// neighbouring SMs computes one 256 x 256 tile.  Each block loads its 128 rows of X and its 128 of
// the tile's 256 rows of Y (a third less shared-memory fill per flop than 128 x 256 tiles of
// single blocks), the leader (rank 0) issues tcgen05.mma.cta_group::2 instructions of 256 x 256 x 16
// that read both blocks' shared memory and accumulate each block's 128 rows in its own tensor
// memory; both blocks' four epilogue warps read their halves back.  Barriers: the TMA loads of
// both blocks complete on the LEADER's full barrier (no multicast of data; the barrier operand is
// the leader's, which cta_group::2 loads allow); a commit with cluster multicast frees a stage,
// and publishes an accumulator, in both blocks; the peer's epilogue threads arrive on the
// leader's accumulator-empty barrier through the cluster's shared window.  Persistent: cluster c
// walks tiles c, c + clusters, ...; two accumulators (2 x 256 columns) as in the kernel above.
// How a cluster of the pair kernel walks through its work.  Whole units: unit u is tile
// u % whole_tiles over K range u / whole_tiles (one range unless K is cut by plan), taken round
// robin, cluster c the units c, c + clusters, ...  Ahead of them, when the host found that the last
// round of whole tiles would leave most clusters idle for long, the TAIL: the last tail_tiles tiles are
// cut along K into segments that all clusters share, in such a way that clusters which work at the same
// time walk the SAME range of K in different tiles, as they do in a round of whole tiles (neighbours then
// find each other's operand tiles in L2; clusters that start at scattered K offsets fetch everything from
// memory, which is slower than leaving clusters idle).  The first tail_p * tail_tiles clusters ("main")
// take K blocks [0, tail_x) of a tile, cut into tail_p equal slices: cluster c the slice c / tail_tiles
// of tail tile c % tail_tiles.  The other clusters ("helpers", H of them) take the rest [tail_x, K blocks)
// of tail tiles h, h + H, h + 2H, ...  The host chooses tail_x so that both kinds end together.  A
// segment's 32-bit partial tile goes to the workspace, slot (tail tile, segment, block of the pair);
// the block whose segment is the LAST of a tile to arrive (a counter per tile and block of the pair,
// which that block also puts back to zero) adds the tile's partial tiles in the order of their K ranges
// and stores the result.  Nothing waits for anything: no flag is spun on.
struct PairUnit {
    int tile, kb0, nkb, range, seg;
    bool partial;
};
struct PairWalk {
    int unit, clusters, whole_units, whole_tiles, kb_per_split, k_blocks;
    int tail_tiles, tail_p, tail_x, tail_tile, tail_step, tail_seg, tail_kb0, tail_nkb;
    __device__ PairWalk(int cluster, int clusters_, int num_tiles, int splits, int kb_per_split_, int k_blocks_, int tail_tiles_, int tail_p_, int tail_x_)
        : unit(cluster), clusters(clusters_), whole_units((num_tiles - tail_tiles_) * splits), whole_tiles(num_tiles - tail_tiles_),
          kb_per_split(kb_per_split_), k_blocks(k_blocks_), tail_tiles(tail_tiles_), tail_p(tail_p_), tail_x(tail_x_)
    {
        const int mains = tail_p * tail_tiles;
        if (cluster < mains) {                 // one slice of [0, tail_x) of one tail tile
            const int slice = cluster / tail_tiles;
            tail_tile = cluster % tail_tiles;
            tail_step = tail_tiles;            // no second segment
            tail_seg = slice;
            tail_kb0 = (int)((long long)slice * tail_x / tail_p);
            tail_nkb = (int)((long long)(slice + 1) * tail_x / tail_p) - tail_kb0;
        } else {                               // the rest [tail_x, k_blocks) of every (clusters - mains)-th tail tile
            tail_tile = tail_x < k_blocks ? cluster - mains : tail_tiles;
            tail_step = clusters - mains;
            tail_seg = tail_p;
            tail_kb0 = tail_x;
            tail_nkb = k_blocks - tail_x;
        }
    }
    __device__ bool next(PairUnit& u)
    {
        // the tail's segments come FIRST: the sums over their partial tiles (round trips to L2, by the epilogue warps
        // of whichever block arrives last) then run beside the main loops of the whole tiles that follow, not after
        // everything else as the kernel's last act
        if (tail_tile < tail_tiles) {
            u.tile = whole_tiles + tail_tile;
            u.range = 0;
            u.kb0 = tail_kb0;
            u.nkb = tail_nkb;
            u.partial = true;
            u.seg = tail_seg;
            tail_tile += tail_step;
            return true;
        }
        if (unit < whole_units) {
            u.tile = unit % whole_tiles;
            u.range = unit / whole_tiles;
            u.kb0 = u.range * kb_per_split;
            u.nkb = (k_blocks < u.kb0 + kb_per_split ? k_blocks : u.kb0 + kb_per_split) - u.kb0;
            u.partial = false;
            u.seg = 0;
            unit += clusters;
            return true;
        }
        return false;
    }
};
constexpr int PAIR_TAIL_MAX_TILES = 512;
__device__ int g_pair_tail_count[2 * PAIR_TAIL_MAX_TILES];   // [tail tile][block of the pair]: segments of the tile that have arrived

constexpr int PAIR_STAGES = 6;
constexpr int PAIR_X_BYTES = BM * BK * 2;                    // 128 rows of X
constexpr int PAIR_STAGE_BYTES = 2 * PAIR_X_BYTES;           // and 128 rows of Y
constexpr size_t PAIR_SMEM = (size_t)PAIR_STAGES * PAIR_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

template <typename TC, int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, TC* __restrict__ out,
                         long long ld, int x_rows, int y_rows, int k_blocks, int x_tiles, int num_tiles, int splits, int kb_per_split,
                         long long split_stride, int tail_tiles, int tail_p, int tail_x, float* __restrict__ workspace, int* status)
{
    // splits > 1 (few tiles, 512 tokens or so): a work unit is one tile over one range of kb_per_split K blocks; unit u is
    // tile u % num_tiles of range u / num_tiles, and its 32-bit partial tile goes to out + range * split_stride (the
    // caller sums the ranges in order).  With one range a unit is a whole tile.
    constexpr int BN = 256;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* tiles = smem;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + (size_t)PAIR_STAGES * PAIR_STAGE_BYTES);   // the leader's are used
    uint64_t* empty_bar = full_bar + PAIR_STAGES;   // every block's own
    uint64_t* acc_full = empty_bar + PAIR_STAGES;   // [2] every block's own
    uint64_t* acc_empty = acc_full + 2;             // [2] the leader's are used: 256 arrivals
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* tail_last = reinterpret_cast<volatile int*>(tmem_slot + 2);   // this block's segment was the last of its tile to arrive

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const int cluster = blockIdx.x >> 1, clusters = gridDim.x >> 1;
    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            mbar_init(full_bar + s, 1);
            mbar_init(empty_bar + s, 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(acc_full + b, 1);
            mbar_init(acc_empty + b, 256);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, 2u * BN);
    fence_before_sync();
    __syncthreads();
    cluster_sync();   // both blocks' barriers are initialised and their tensor memory is allocated before either is used from the other side
    fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    pdl_launch_dependents();
    if (warp == 0) {
        if (lane == 0) {
            long long g = 0;
            bool ok = true, first = true;
            PairWalk walk(cluster, clusters, num_tiles, splits, kb_per_split, k_blocks, tail_tiles, tail_p, tail_x);
            PairUnit u;
            while (ok && walk.next(u)) {
                const int tile = u.tile, kb0 = u.kb0, nkb = u.nkb;
                const int x0 = (tile % x_tiles) * (2 * BM) + (int)rank * BM, y0 = (tile / x_tiles) * BN + (int)rank * (BN / 2);
                int kb = 0;
                if (first) {
                    // the weights (Y) of the first stages are requested before the wait for the kernels ahead in the stream
                    const int pre = min(nkb, PAIR_STAGES);
                    for (int i = 0; i < pre; ++i) {
                        if (rank == 0) mbar_expect_tx(full_bar + i, 2 * PAIR_STAGE_BYTES);
                        tma_load_2d_pair(smem_u32(tiles + (size_t)i * PAIR_STAGE_BYTES + PAIR_X_BYTES), &map_y, (kb0 + i) * BK, y0, map_to_rank(smem_u32(full_bar + i), 0));
                    }
                    pdl_wait();
                    for (int i = 0; i < pre; ++i)
                        tma_load_2d_pair(smem_u32(tiles + (size_t)i * PAIR_STAGE_BYTES), &map_x, (kb0 + i) * BK, x0, map_to_rank(smem_u32(full_bar + i), 0));
                    kb = pre;
                    g = pre;
                    first = false;
                }
                for (; kb < nkb; ++kb, ++g) {
                    const int s = (int)(g % PAIR_STAGES);
                    const uint32_t phase = (uint32_t)(g / PAIR_STAGES) & 1;
                    if (g >= PAIR_STAGES && !mbar_wait(empty_bar + s, phase ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* xs = tiles + (size_t)s * PAIR_STAGE_BYTES;
                    if (rank == 0) mbar_expect_tx(full_bar + s, 2 * PAIR_STAGE_BYTES);   // both blocks' bytes
                    const uint32_t leader_full = map_to_rank(smem_u32(full_bar + s), 0);
                    tma_load_2d_pair(smem_u32(xs), &map_x, (kb0 + kb) * BK, x0, leader_full);
                    tma_load_2d_pair(smem_u32(xs + PAIR_X_BYTES), &map_y, (kb0 + kb) * BK, y0, leader_full);
                }
            }
            if (first) pdl_wait();
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = instr_desc_bf16(2 * BM, BN, false, false);
            long long g = 0;
            int i = 0;
            bool ok = true;
            PairWalk walk(cluster, clusters, num_tiles, splits, kb_per_split, k_blocks, tail_tiles, tail_p, tail_x);
            PairUnit u;
            for (; ok && walk.next(u); ++i) {
                const int nkb = u.nkb;
                const int buf = i & 1;
                const uint32_t aph = (uint32_t)(i >> 1) & 1;
                if (i >= 2) ok = mbar_wait(acc_empty + buf, aph ^ 1, abort_flag);   // both blocks' epilogues have read this buffer's last tile
                if (!ok) break;
                fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t)buf * BN;
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = (int)(g % PAIR_STAGES);
                    const uint32_t phase = (uint32_t)(g / PAIR_STAGES) & 1;
                    ok = mbar_wait(full_bar + s, phase, abort_flag);
                    if (!ok) break;
                    fence_after_sync();
                    const uint8_t* xs = tiles + (size_t)s * PAIR_STAGE_BYTES;
                    const uint64_t dx = desc_k_major(smem_u32(xs)), dy = desc_k_major(smem_u32(xs + PAIR_X_BYTES));
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        const uint64_t adv = (uint64_t)((k * UMMA_K * 2) >> 4);
                        umma_pair(acc, dx + adv, dy + adv, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    umma_commit_pair(empty_bar + s);
                }
                if (ok) umma_commit_pair(acc_full + buf);
            }
        }
    } else {
        const int quarter = warp & 3;
        pdl_wait();   // the output buffer may still be in use by a kernel ahead in the stream
        int i = 0;
        bool ok = true;
        PairWalk walk(cluster, clusters, num_tiles, splits, kb_per_split, k_blocks, tail_tiles, tail_p, tail_x);
        PairUnit u;
        const int whole_tiles = num_tiles - tail_tiles;
        for (; ok && walk.next(u); ++i) {
            const int tile = u.tile;
            TC* unit_out = out + (size_t)u.range * split_stride;
            const int buf = i & 1;
            const uint32_t aph = (uint32_t)(i >> 1) & 1;
            const int x0 = (tile % x_tiles) * (2 * BM) + (int)rank * BM, y0 = (tile / x_tiles) * BN;
            ok = mbar_wait(acc_full + buf, aph, abort_flag);
            if (!ok) break;
            fence_after_sync();
            const int row = quarter * 32 + lane;
            const int x = x0 + row;
            if (!u.partial) {
#pragma unroll 1
                for (int c = 0; c < BN; c += 32) {
                    uint32_t r[32];
                    tmem_load<32>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c), r);
                    tmem_wait_ld();
                    store_chunk_normal<TC, EPI>(unit_out, ld, x, y0 + c, x_rows, y_rows, r);
                }
                fence_before_sync();
                if (rank == 0) mbar_arrive(acc_empty + buf);
                else mbar_arrive_cluster(map_to_rank(smem_u32(acc_empty + buf), 0));
                continue;
            }
            // a segment of a tail tile: the partial tile goes to the workspace, and the accumulator is free again
            const int tile_rel = tile - whole_tiles;
            const int segments = tail_p + (tail_x < k_blocks ? 1 : 0);   // of every tail tile, in the order of their K ranges
            float* mine = workspace + (((size_t)tile_rel * (tail_p + 1) + u.seg) * 2 + rank) * STREAM_TILE_FLOATS;
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                uint32_t r[32];
                tmem_load<32>(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * BN + c), r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    __stcg(reinterpret_cast<float4*>(mine + partial_index(c, j, row)),
                           make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
            }
            fence_before_sync();
            if (rank == 0) mbar_arrive(acc_empty + buf);
            else mbar_arrive_cluster(map_to_rank(smem_u32(acc_empty + buf), 0));
            __threadfence();
            epilogue_barrier();
            if (row == 0) {
                const int arrived = atomicAdd(&g_pair_tail_count[tile_rel * 2 + (int)rank], 1);
                *tail_last = arrived == segments - 1 ? 1 : 0;
            }
            epilogue_barrier();
            const bool last = *tail_last != 0;
            epilogue_barrier();   // everybody has read the flag before a later segment's arrival may write it again
            if (!last) continue;
            __threadfence();
#pragma unroll 1
            for (int c = 0; c < BN; c += 32) {
                float4 sum[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) sum[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int sg = 0; sg < segments; sg += 2) {   // two segments' loads in flight: the sums are bound by the round trips to L2
                    const float* first = workspace + (((size_t)tile_rel * (tail_p + 1) + sg) * 2 + rank) * STREAM_TILE_FLOATS;
                    const bool two = sg + 1 < segments;
                    const float* second = two ? first + 2 * (size_t)STREAM_TILE_FLOATS : first;
                    float4 v[8], w[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) v[j] = __ldcg(reinterpret_cast<const float4*>(first + partial_index(c, j, row)));
#pragma unroll
                    for (int j = 0; j < 8; ++j) w[j] = __ldcg(reinterpret_cast<const float4*>(second + partial_index(c, j, row)));
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        sum[j].x += v[j].x;
                        sum[j].y += v[j].y;
                        sum[j].z += v[j].z;
                        sum[j].w += v[j].w;
                        if (two) {
                            sum[j].x += w[j].x;
                            sum[j].y += w[j].y;
                            sum[j].z += w[j].z;
                            sum[j].w += w[j].w;
                        }
                    }
                }
                uint32_t r[32];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    r[4 * j] = __float_as_uint(sum[j].x);
                    r[4 * j + 1] = __float_as_uint(sum[j].y);
                    r[4 * j + 2] = __float_as_uint(sum[j].z);
                    r[4 * j + 3] = __float_as_uint(sum[j].w);
                }
                store_chunk_normal<TC, EPI>(unit_out, ld, x, y0 + c, x_rows, y_rows, r);
            }
            if (row == 0) g_pair_tail_count[tile_rel * 2 + (int)rank] = 0;   // for the next product: nobody else touches it in this one
        }
    }

    fence_before_sync();
    __syncthreads();
    if (*abort_flag) {
        if (threadIdx.x == 0) {
            const unsigned long long t0 = global_timer();
            while (global_timer() - t0 < 2000000ull) { }
            report_status(status, SPY_STATUS_WAIT_TIMEOUT, (int)blockIdx.x);
        }
        __syncthreads();
    }
    cluster_sync();   // neither block leaves (and frees tensor memory the pair shares) while the other may still use it
    if (warp == 1) {
        fence_after_sync();
        tmem_dealloc_pair(tmem_base, 2u * BN);
    }
}

// Sums the splits of a scratch buffer in ascending order and stores the output type.
template <typename TC>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, TC* __restrict__ out, long long elems, int splits)
{
    pdl_enter();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < elems; i += (long long)gridDim.x * blockDim.x) {
        float acc = partial[i];
        for (int s = 1; s < splits; ++s) acc += partial[(size_t)s * elems + i];
        out[i] = from_f32<TC>(acc);
    }
}

// A [rows, K] bfloat16 matrix with K contiguous; box = 64 columns x box_rows rows, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, long long rows, long long K, long long ld, int box_rows)
{
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) SPY_FAIL("gemm_tcgen05: cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) SPY_FAIL("gemm_tcgen05: cuTensorMapEncodeTiled failed with code %d (rows %lld, K %lld, ld %lld)", (int)r, rows, K, ld);
    return 0;
}

// The partial products [splits][M][N] of the scratch summed in order into C.
static int reduce_splits(const float* scratch, void* C, int c_dtype, long long ldc, int M, int N, int splits, cudaStream_t stream)
{
    const long long elems = (long long)M * N;
    if (ldc != N) SPY_FAIL("gemm_tcgen05: split-K needs a contiguous output (ldc %lld, N %d)", ldc, N);
    long long blocks = (elems + 255) / 256;
    if (blocks > spy_sm_count() * 8) blocks = spy_sm_count() * 8;
    if (c_dtype == SPY_F32) spy_launch(splitk_reduce_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, scratch, (float*)C, elems, splits);
    else spy_launch(splitk_reduce_kernel<bf16>, dim3((int)blocks), dim3(256), 0, stream, scratch, (bf16*)C, elems, splits);
    SPY_CHECK_LAUNCH("gemm_tcgen05 split-K reduce");
    return 0;
}

template <int BN, typename TC, int EPI>
static int launch(const CUtensorMap& mx, const CUtensorMap& my, void* out, long long ld, long long split_stride, int x_rows, int y_rows,
                  int k_blocks, int splits, int tile_rows, int* status, cudaStream_t stream, const void* next_weights, long long next_bytes)
{
    using T = Tile<BN>;
    auto kernel = gemm_tcgen05_kernel<BN, TC, EPI>;
    SPY_ONCE_PER_DEVICE {
        SPY_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)T::SMEM));
    }
    const int per_split = (k_blocks + splits - 1) / splits;
    dim3 grid((y_rows + BN - 1) / BN, (x_rows + tile_rows - 1) / tile_rows, splits);   // token tiles fastest
    if (grid.y > 65535 || grid.z > 65535) SPY_FAIL("gemm_tcgen05: the grid %u x %u x %u exceeds the launch limits", grid.x, grid.y, grid.z);
    spy_launch(kernel, grid, dim3(NUM_THREADS), T::SMEM, stream, mx, my, (TC*)out, ld, split_stride, x_rows, y_rows, k_blocks, per_split, tile_rows,
               status, (const uint8_t*)next_weights, next_bytes);
    SPY_CHECK_LAUNCH("gemm_tcgen05");
    return 0;
}

}  // namespace

namespace {

// The plan of a product: the kernel it runs on (choose_kind), how many ways K is split and how many weight rows a block takes.
// Pairs and single blocks (many tokens): 256 x 256 or 128 x 256 tiles; K is cut into ranges by plan only for pairs with
// few tiles (the single-block kernel shares K blocks out itself when there are fewer tiles than SMs).
// The swapped kernel (few tokens: decoding; the weights sit in the instruction's M slot, two blocks share an
// SM; the token tile is 16, 32, 64 or 128 tokens (65 to 128 tokens in ONE tile of 128: against two tiles of
// 64, which read every weight tile from L2 twice, gate‖up of the 8B shape 53 -> 42 us, down 26 -> 24, of the
// 14B shape 75 -> 62 and 48 -> 38); more than 128 tokens, where the pairs find too little work, are two token
// tiles whose blocks start side by side and share every weight tile through L2, so the plan fills the slots
// divided by the token tiles):
// the product is bound by reading the weights, so what counts is that all 2 x SMs block
// slots stream at once and end together.  When 128-row tiles times the splits would not fill
// the slots, the tile takes fewer rows (a multiple of 4, at least 64: the TMA box shrinks, the
// tensor core still multiplies 128 rows and the spare ones are dropped), so that tiles x splits
// comes as close to the slots as it can; among the ways to split K the cheapest by a small
// model wins (work per block, a fixed cost per block, a cost per split for the partial sums
// the consumer has to add).  The choice depends on N, K and the class of M only.
// SPYINFER_GEMM_PAIRS=0 in the environment keeps the products for many tokens on single blocks.
bool pair_kernel_enabled()
{
    const char* e = getenv("SPYINFER_GEMM_PAIRS");   // read at every call: a test may switch it
    return !(e != nullptr && e[0] == '0');
}

bool tail_sharing_enabled()
{
    const char* e = getenv("SPYINFER_GEMM_TAIL");   // read at every call: a test may switch it
    return !(e != nullptr && e[0] == '0');
}

// K blocks of one cluster's time that sharing the last round must save to be used
// (SPYINFER_GEMM_TAIL_MIN in the environment overrides it: tests use 0 to reach the path at every size).
long long tail_sharing_threshold()
{
    const char* e = getenv("SPYINFER_GEMM_TAIL_MIN");
    return e != nullptr ? atoll(e) : 8;
}

// How the left-over tiles of the pair kernel's last round are cut (see PairWalk): p main clusters a tile share K blocks
// [0, x) in equal slices, the other clusters take [x, k_blocks) of the tiles in turns; x is where both kinds end together,
// a helper's turn counted with what its hand-over costs beside the K blocks themselves (the accumulator's way to the
// workspace and the arrival: about TAIL_TURN_COST K blocks of time; with short turns the helpers ended last by far).
// A segment has at least 8 K blocks.  saved: K blocks of one cluster's time that the last round no longer takes.
struct TailPlan {
    int p, x;
    long long saved;
};
constexpr int TAIL_TURN_COST = 16;
TailPlan plan_tail(int tiles, int clusters, int k_blocks)
{
    TailPlan t;
    t.p = clusters / tiles;
    while (t.p > 1 && k_blocks / t.p < 8) --t.p;
    const int helpers = clusters - t.p * tiles;
    const long long turns = helpers > 0 ? (tiles + helpers - 1) / helpers : 0;
    t.x = k_blocks;
    if (helpers > 0) {
        // x / p = turns * (k_blocks - x + cost)
        const long long x = (long long)t.p * turns * (k_blocks + TAIL_TURN_COST) / (1 + t.p * turns);
        if (x < k_blocks && k_blocks - x >= 8 && x / t.p >= 8) t.x = (int)x;
    }
    const long long main_time = (t.x + t.p - 1) / t.p, helper_time = t.x < k_blocks ? turns * (k_blocks - t.x + TAIL_TURN_COST) : 0;
    t.saved = k_blocks - (main_time > helper_time ? main_time : helper_time);
    return t;
}

enum Kind { SWAPPED, SINGLE, PAIRS };   // the kernel a product runs on
// The swapped kernel's token tile (the instruction's N): 16, 32, 64 or 128 tokens, the smallest that holds them all.
static inline int token_tile(int M) { return M <= 16 ? 16 : (M <= 32 ? 32 : (M <= 64 ? 64 : 128)); }
struct Plan {
    int splits, tile_rows;
    Kind kind;
};

static inline int pair_min_tiles() { return (spy_sm_count() / 2 + 1) / 2; }   // whole 256 x 256 tiles occupy at least half of the clusters (SMs / 2) from here on

// Which kernel a product runs on.  Up to 128 tokens: the swapped kernel (weights in the instruction's M slot, one or
// two token tiles of 64).  Beyond: pairs of blocks on 256 x 256 tiles where they find enough work (whole tiles for
// at least half of the clusters, or, where K may be cut into ranges, at least 8 tiles), else the swapped kernel up
// to 256 tokens and single blocks on 128 x 256 tiles above.  129 to 256 tokens (one row of 256-token tiles; a third and
// fourth token tile of the swapped kernel would read every weight tile from L2 again: measured at 256 tokens, 8B
// sizes q‖k‖v 26 -> 21 us, gate‖up 75 -> 51, down 37 -> 29; 14B sizes gate‖up 127 -> 79, down 88 -> 48; at 128 tokens
// the swapped kernel is still ahead).  257 to 511 tokens (a third or fourth 128-token tile that pairs round up to 512):
// pairs when the single blocks would have fewer tiles than SMs (their shared K blocks cost more than the pairs' K
// ranges: at 320 to 448 tokens q‖k‖v 33-40 -> 28-29 us, o 33-36 -> 20, down 54-78 -> 42-44), and otherwise when the
// pairs' rounds of tiles, the last one counted by what sharing it out leaves of it, are no more than the single
// blocks' (gate‖up at 320 and 384 tokens: 288 tiles are two rounds of single blocks = 67-69 us, 192 tiles 2.6 rounds
// of pairs = 79-81 us; at 448 tokens three rounds either way, 88 against 83 us).  From 512 tokens on: pairs.
Kind choose_kind(int M, int N, bool may_split)
{
    if (M <= 2 * 64) return SWAPPED;
    const Kind other = M <= 256 ? SWAPPED : SINGLE;
    if (!pair_kernel_enabled()) return other;
    const int sms = spy_sm_count();
    const long long y_tiles = (N + 255) / 256;
    const long long tiles1 = (long long)((M + BM - 1) / BM) * y_tiles, tiles2 = (long long)((M + 2 * BM - 1) / (2 * BM)) * y_tiles;
    if (!(tiles2 >= pair_min_tiles() || (may_split && tiles2 >= 8))) return other;
    if (M <= 256 || M >= 512 || tiles1 < sms) return PAIRS;
    const long long clusters = sms / 2;
    const long long r1 = (tiles1 + sms - 1) / sms;
    const long long r2 = (tiles2 * 10 - 3 * clusters + 10 * clusters - 1) / (10 * clusters);   // ceil(tiles2 / clusters - 0.3)
    return r2 <= r1 ? PAIRS : SINGLE;
}

Plan make_plan(int M, int N, int K, bool may_split)
{
    const int k_blocks = (K + BK - 1) / BK;
    Plan best = {1, BM, choose_kind(M, N, may_split)};
    if (best.kind == PAIRS && may_split) {
        // a few hundred tokens on pairs of blocks: with too few 256 x 256 tiles for the clusters (o and down at the 8B
        // shape: 32), K is cut into two to four ranges, so that tiles x ranges occupy most of the clusters (SMs / 2); the
        // partial tiles are summed by the caller or by the reduce kernel.  At least 16 K blocks a range.
        const long long tiles = (long long)((M + 2 * BM - 1) / (2 * BM)) * ((N + 255) / 256);
        if (tiles >= 8 && tiles < pair_min_tiles()) {
            int s = (int)(spy_sm_count() / 2 / tiles);
            if (s > 4) s = 4;
            while (s > 1 && (k_blocks / s < 16 || (k_blocks + (k_blocks + s - 1) / s - 1) / ((k_blocks + s - 1) / s) != s)) --s;
            best.splits = s;
            if (s == 1) best.kind = M <= 256 ? SWAPPED : SINGLE;   // K is too short for ranges: too few tiles for the clusters
        }
        if (best.kind == PAIRS) return best;
    }
    if (best.kind != SWAPPED) return best;   // many tokens: the persistent kernels share the work out themselves (stream-K)
    const int token_tiles = (M + token_tile(M) - 1) / token_tile(M);   // more than 128 tokens: two token tiles share every weight tile
    const int slots = 2 * spy_sm_count() / (token_tiles > 0 ? token_tiles : 1);
    if ((N + BM - 1) / BM >= slots) return best;   // more 128-row tiles than slots: they spread evenly as they are
    int most = may_split ? (k_blocks / 4 > 0 ? k_blocks / 4 : 1) : 1;
    if (most > 16) most = 16;
    double best_cost = 0;
    for (int s = 1; s <= most; ++s) {
        const int per = (k_blocks + s - 1) / s;
        if ((k_blocks + per - 1) / per != s) continue;   // would leave an empty trailing split
        int rows = BM;
        const long long full = (long long)((N + BM - 1) / BM) * s;
        if (full < slots) {
            rows = ((N + slots / s - 1) / (slots / s) + 3) / 4 * 4;   // the fewest rows with which the tiles still fit the slots
            if (rows < 64) rows = 64;
            if (rows > BM) rows = BM;
        }
        const long long ctas = (long long)((N + rows - 1) / rows) * s;
        const double waves = ctas <= slots ? 1.0 : (ctas <= 2 * slots ? 2.0 : (double)ctas / slots + 0.5);
        const double cost = waves * ((double)rows * per + 344.0) + 20.0 * s;
        if (s == 1 || cost < best_cost) {
            best_cost = cost;
            best.splits = s;
            best.tile_rows = rows;
        }
    }
    return best;
}

}  // namespace

// How many splits of K a product of this shape uses, and the floats of scratch it needs.
// A plan that would need more than scratch_limit floats falls back to one pass over K.
extern "C" int spy_gemm_tcgen05_plan(int M, int N, int K, long long scratch_limit, int* splits_out, long long* scratch_floats_out)
{
    Plan plan = make_plan(M, N, K, true);
    long long need = plan.splits > 1 ? (long long)plan.splits * M * N : 0;
    if (need > scratch_limit) {   // not enough scratch: one pass over K
        plan = make_plan(M, N, K, false);
        need = 0;
    }
    *splits_out = plan.splits;
    *scratch_floats_out = need;
    return 0;
}

// A [M, K] and W [N, K] bfloat16, rows lda/ldw elements apart; C [M, N] of c_dtype, rows ldc
// apart.  scratch: float buffer of at least the plan's size (may be null when it is 0).
// epilogue 1 (SwiGLU): W's rows alternate gate and up rows, C is [M, N / 2], K is not split.
// defer_reduce: when the plan splits K, the partial products stay in scratch as
// [splits][M][N] floats for the consumer to sum (C is not written); *splits_used tells.
// next_weights / next_bytes (may be null / 0; used by products of up to 256 tokens only): memory that a
// later kernel of the stream will read, typically the next product's weights; the blocks ask for it to
// be brought into L2 once their own loads are requested.  16-byte aligned.
extern "C" int spy_gemm_tcgen05_ex(const void* A, long long lda, const void* W, long long ldw, void* C, int c_dtype, long long ldc, int M, int N,
                                   int K, float* scratch, long long scratch_floats, int epilogue, int defer_reduce, int* splits_used,
                                   int* status, cudaStream_t stream, const void* next_weights, long long next_bytes)
{
    if (next_weights == nullptr || next_bytes <= 0 || (reinterpret_cast<uintptr_t>(next_weights) & 15)) {
        next_weights = nullptr;
        next_bytes = 0;
    }
    if (splits_used) *splits_used = 1;
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0) SPY_FAIL("gemm_tcgen05: K %d must be a positive multiple of 8 (16-byte rows for TMA)", K);
    if (lda % 8 != 0 || ldw % 8 != 0) SPY_FAIL("gemm_tcgen05: row strides %lld/%lld must be multiples of 8 elements", lda, ldw);
    if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15)) SPY_FAIL("gemm_tcgen05: operands must be 16-byte aligned");
    if (c_dtype != SPY_F32 && c_dtype != SPY_BF16) SPY_FAIL("gemm_tcgen05: unknown output dtype code %d", c_dtype);
    if (epilogue != 0 && epilogue != 1) SPY_FAIL("gemm_tcgen05: unknown epilogue %d", epilogue);
    if (epilogue == 1 && (N % 2 != 0 || c_dtype != SPY_BF16)) SPY_FAIL("gemm_tcgen05: the SwiGLU epilogue needs an even N and bfloat16 output");
    Plan plan = make_plan(M, N, K, epilogue == 0);
    if (plan.splits > 1 && (scratch == nullptr || (long long)plan.splits * M * N > scratch_floats)) plan = make_plan(M, N, K, false);
    const int splits = plan.splits;
    if (splits_used) *splits_used = splits;
    const int k_blocks = (K + BK - 1) / BK;
    const bool swap = plan.kind == SWAPPED;
    const int bn = swap ? token_tile(M) : 256;
    CUtensorMap mx, my;
    if (swap) {
        if (make_map(&mx, W, N, K, ldw, plan.tile_rows) || make_map(&my, A, M, K, lda, bn)) return 1;
    } else {
        if (make_map(&mx, A, M, K, lda, BM) || make_map(&my, W, N, K, ldw, bn)) return 1;
    }
    const int x_rows = swap ? N : M, y_rows = swap ? M : N;
    void* out = splits > 1 ? (void*)scratch : C;
    const long long ld = splits > 1 ? N : ldc;
    const long long split_stride = splits > 1 ? (long long)M * N : 0;
    const bool f32_out = splits > 1 || c_dtype == SPY_F32;
    // pairs need enough 256 x 256 tiles to occupy at least half of the clusters; smaller products go to single
    // blocks, which share the K blocks of their 128 x 256 tiles out over all SMs
    if (plan.kind == PAIRS) {
        // many tokens, one pass over K, at least two 256-row tiles: pairs of blocks on 256 x 256 tiles
        CUtensorMap my_half;
        if (make_map(&my_half, W, N, K, ldw, BM)) return 1;
        const int x_tiles = (M + 2 * BM - 1) / (2 * BM), y_tiles = (N + 255) / 256;
        const long long num_tiles = (long long)x_tiles * y_tiles;
        if (num_tiles > 0x7fffffffLL) SPY_FAIL("gemm_tcgen05: %lld tiles exceed the kernel's range", num_tiles);
        static int clusters_of_device[SPY_MAX_DEVICES] = {};
        int& clusters_max = clusters_of_device[spy_device()];
        if (clusters_max == 0) {
            SPY_CUDA(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<bf16, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAIR_SMEM));
            SPY_CUDA(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<float, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAIR_SMEM));
            SPY_CUDA(cudaFuncSetAttribute(gemm_tcgen05_pair_kernel<bf16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)PAIR_SMEM));
            const int sms = spy_sm_count();
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(sms / 2 * 2);
            cfg.blockDim = dim3(NUM_THREADS);
            cfg.dynamicSmemBytes = PAIR_SMEM;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 2;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int active = 0;
            SPY_CUDA(cudaOccupancyMaxActiveClusters(&active, gemm_tcgen05_pair_kernel<bf16, 0>, &cfg));
            if (active <= 0) SPY_FAIL("gemm_tcgen05: no cluster of two blocks fits the device");
            clusters_max = active < sms / 2 ? active : sms / 2;
        }
        const long long num_units = num_tiles * splits;
        const int clusters = (int)(num_units < clusters_max ? num_units : clusters_max);
        const int kb_per_split = (k_blocks + splits - 1) / splits;
        if (splits > 1) {
            // ranges of K: 32-bit partial tiles into the scratch, [range][M][N]
            spy_launch_cluster(gemm_tcgen05_pair_kernel<float, 0>, dim3(2 * clusters), dim3(NUM_THREADS), PAIR_SMEM, stream, 2u, mx, my_half, (float*)scratch,
                               (long long)N, M, N, k_blocks, x_tiles, (int)num_tiles, splits, kb_per_split, split_stride, 0, 1, 0, (float*)nullptr, status);
            SPY_CHECK_LAUNCH("gemm_tcgen05 (pairs, K ranges)");
            if (!defer_reduce) {
                if (int rc = reduce_splits(scratch, C, c_dtype, ldc, M, N, splits, stream)) return rc;
            }
            return 0;
        }
        // The last round of whole tiles.  When it would leave clusters idle (the down projections of the larger models
        // are 160 tiles on 74 clusters, a third round for twelve tiles; at 2,048 tokens of the 8B shape 54 of 128 tiles
        // are left over), its tiles are cut along K and shared out over all clusters instead (see PairWalk and plan_tail),
        // through partial tiles in the scratch.  Measured inside whole prompts: 2 to 7 % at the 14B and 32B sizes, nothing
        // lost at the 8B sizes.  Timed alone the gain is smaller than the idle time it removes: under the power cap the
        // idle clusters of a last round lend their share of the power to the busy rounds.
        int tail_tiles = 0, tail_p = 1, tail_x = 0;
        const long long left = num_tiles % clusters_max;
        if (tail_sharing_enabled() && num_tiles > clusters_max && left > 0 && left <= PAIR_TAIL_MAX_TILES && scratch != nullptr) {
            const TailPlan tp = plan_tail((int)left, clusters_max, k_blocks);
            if (tp.saved >= tail_sharing_threshold() && scratch_floats >= left * (tp.p + 1) * 2 * (long long)STREAM_TILE_FLOATS) {
                tail_tiles = (int)left;
                tail_p = tp.p;
                tail_x = tp.x;
            }
        }
        if (epilogue == 1)
            spy_launch_cluster(gemm_tcgen05_pair_kernel<bf16, 1>, dim3(2 * clusters), dim3(NUM_THREADS), PAIR_SMEM, stream, 2u, mx, my_half, (bf16*)C, ldc,
                               M, N, k_blocks, x_tiles, (int)num_tiles, 1, k_blocks, 0LL, tail_tiles, tail_p, tail_x, scratch, status);
        else if (c_dtype == SPY_F32)
            spy_launch_cluster(gemm_tcgen05_pair_kernel<float, 0>, dim3(2 * clusters), dim3(NUM_THREADS), PAIR_SMEM, stream, 2u, mx, my_half, (float*)C, ldc,
                               M, N, k_blocks, x_tiles, (int)num_tiles, 1, k_blocks, 0LL, tail_tiles, tail_p, tail_x, scratch, status);
        else
            spy_launch_cluster(gemm_tcgen05_pair_kernel<bf16, 0>, dim3(2 * clusters), dim3(NUM_THREADS), PAIR_SMEM, stream, 2u, mx, my_half, (bf16*)C, ldc,
                               M, N, k_blocks, x_tiles, (int)num_tiles, 1, k_blocks, 0LL, tail_tiles, tail_p, tail_x, scratch, status);
        SPY_CHECK_LAUNCH("gemm_tcgen05 (pairs)");
        return 0;
    }
    if (!swap && splits == 1) {
        // many tokens, one pass over K: the persistent kernel (one block per SM)
        const int num_sms = spy_sm_count();
        const int x_tiles = (M + BM - 1) / BM, y_tiles = (N + 255) / 256;
        const long long num_tiles = (long long)x_tiles * y_tiles;
        if (num_tiles > 0x7fffffffLL) SPY_FAIL("gemm_tcgen05: %lld tiles exceed the kernel's range", num_tiles);
        int grid = (int)(num_tiles < num_sms ? num_tiles : num_sms);
        // stream-K when the scratch holds a partial tile for every block: the K blocks of all tiles are
        // shared out evenly over as many blocks as there are SMs (fewer for very small products)
        int per_block = 0, stream_tiles = 0;
        long long blocks = num_sms;
        if (blocks > STREAM_MAX_BLOCKS) blocks = STREAM_MAX_BLOCKS;
        if (scratch != nullptr && blocks > scratch_floats / STREAM_TILE_FLOATS) blocks = scratch_floats / STREAM_TILE_FLOATS;
        if (scratch != nullptr && blocks >= 1 && num_tiles < blocks) {
            // Fewer tiles than SMs: their K blocks are shared out, so that a block gets at least a quarter of a
            // tile and STREAM_MIN_KB K blocks.  With more tiles than SMs whole tiles stay faster, although the
            // last round is not full (measured at 2,048 tokens: 55.7 against 62 to 64 microseconds for N = K =
            // 4096): the blocks of a round walk K in step, so the tiles of a row or column block meet in L2,
            // and blocks with shares start at different K and do not.
            stream_tiles = (int)num_tiles;
            const long long total = (long long)stream_tiles * k_blocks;
            long long least = k_blocks / 4 > STREAM_MIN_KB ? k_blocks / 4 : STREAM_MIN_KB;
            if (least > k_blocks) least = k_blocks;
            if (total / blocks < least) blocks = total / least > 0 ? total / least : 1;
            per_block = (int)((total + blocks - 1) / blocks);
            grid = (int)((total + per_block - 1) / per_block);
            if (num_tiles > stream_tiles && grid < blocks) grid = (int)blocks;   // whole tiles behind the shared ones: every block takes some
        }
        SPY_ONCE_PER_DEVICE {
            SPY_CUDA(cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<bf16, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WideTile::SMEM));
            SPY_CUDA(cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<float, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WideTile::SMEM));
            SPY_CUDA(cudaFuncSetAttribute(gemm_tcgen05_persistent_kernel<bf16, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)WideTile::SMEM));
        }
        if (epilogue == 1)
            spy_launch(gemm_tcgen05_persistent_kernel<bf16, 1>, dim3(grid), dim3(NUM_THREADS), WideTile::SMEM, stream, mx, my, (bf16*)C, ldc, M, N,
                       k_blocks, x_tiles, (int)num_tiles, stream_tiles, per_block, scratch, status);
        else if (c_dtype == SPY_F32)
            spy_launch(gemm_tcgen05_persistent_kernel<float, 0>, dim3(grid), dim3(NUM_THREADS), WideTile::SMEM, stream, mx, my, (float*)C, ldc, M, N,
                       k_blocks, x_tiles, (int)num_tiles, stream_tiles, per_block, scratch, status);
        else
            spy_launch(gemm_tcgen05_persistent_kernel<bf16, 0>, dim3(grid), dim3(NUM_THREADS), WideTile::SMEM, stream, mx, my, (bf16*)C, ldc, M, N,
                       k_blocks, x_tiles, (int)num_tiles, stream_tiles, per_block, scratch, status);
        SPY_CHECK_LAUNCH("gemm_tcgen05 (persistent)");
        return 0;
    }
    if (!swap) SPY_FAIL("gemm_tcgen05: no kernel was chosen for M=%d N=%d K=%d (splits %d)", M, N, K, splits);
    int rc;
#define SPY_LAUNCH(BN_)                                                                                                             \
    rc = epilogue == 1 ? launch<BN_, bf16, 1>(mx, my, out, ld, split_stride, x_rows, y_rows, k_blocks, splits, plan.tile_rows, status, stream, next_weights, next_bytes)   \
         : f32_out     ? launch<BN_, float, 0>(mx, my, out, ld, split_stride, x_rows, y_rows, k_blocks, splits, plan.tile_rows, status, stream, next_weights, next_bytes)  \
                       : launch<BN_, bf16, 0>(mx, my, out, ld, split_stride, x_rows, y_rows, k_blocks, splits, plan.tile_rows, status, stream, next_weights, next_bytes)
    if (bn == 16) SPY_LAUNCH(16);
    else if (bn == 32) SPY_LAUNCH(32);
    else if (bn == 128) SPY_LAUNCH(128);
    else SPY_LAUNCH(64);
#undef SPY_LAUNCH
    if (rc) return rc;
    if (splits > 1 && !defer_reduce) return reduce_splits(scratch, C, c_dtype, ldc, M, N, splits, stream);
    return 0;
}


// The plain product: no epilogue, partial products summed before it returns.
extern "C" int spy_gemm_tcgen05(const void* A, long long lda, const void* W, long long ldw, void* C, int c_dtype, long long ldc, int M, int N,
                                int K, float* scratch, long long scratch_floats, int* status, cudaStream_t stream)
{
    return spy_gemm_tcgen05_ex(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, scratch, scratch_floats, 0, 0, nullptr, status, stream, nullptr, 0);
}

// ---------------------------------------------------------------------------------------------
// After a wait ran out (status word SPY_STATUS_WAIT_TIMEOUT) the flags by which the blocks of a
// product with shared K blocks tell one another that a partial tile is ready may be left raised:
// the owner that gave up did not lower them.  The next such product would then add partial tiles
// that are not there yet.  Call this before the next product on that device; it lowers all flags,
// in stream order.  The flags are one array per device for the whole library (this entry point,
// spy_gemm_tcgen05_ex and spy_gemm_tcgen05_static_scratch alike), so products that share K blocks
// (more than 256 tokens and fewer tiles than SMs) must be ordered by their streams, not overlap.
extern "C" int spy_gemm_tcgen05_reset(cudaStream_t stream)
{
    void* flags = nullptr;
    SPY_CUDA(cudaGetSymbolAddress(&flags, g_stream_flags));
    SPY_CUDA(cudaMemsetAsync(flags, 0, sizeof(int) * STREAM_MAX_BLOCKS, stream));
    SPY_CUDA(cudaGetSymbolAddress(&flags, g_pair_tail_count));   // the counters of the pair kernel's tail tiles, for the same reason
    SPY_CUDA(cudaMemsetAsync(flags, 0, sizeof(int) * 2 * PAIR_TAIL_MAX_TILES, stream));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Self-test of the bounded wait that every tensor-core kernel of this library relies on: one warp
// waits on an mbarrier at which nothing ever arrives, with a limit of limit_ns.  The wait must give
// up after the limit, raise the abort flag and return; the kernel then reports
// SPY_STATUS_WAIT_TIMEOUT through the status word exactly as the products and attention kernels
// do, stores how long thread 0 waited, and ends.  It holds no tensor memory and starts no copy.
// Limits above 100 ms are refused: the test is meant to cost a millisecond.
namespace {
__global__ void wait_selftest_kernel(unsigned long long limit_ns, int* status, unsigned long long* waited_ns)
{
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    const unsigned long long t0 = global_timer();
    const bool ok = mbar_wait(&bar, 0, &abort_flag, limit_ns);
    const unsigned long long waited = global_timer() - t0;
    __syncthreads();
    if (threadIdx.x == 0) {
        if (waited_ns != nullptr) *waited_ns = waited;
        if (!ok || abort_flag) report_status(status, SPY_STATUS_WAIT_TIMEOUT, -1);
    }
}
}  // namespace

extern "C" int spy_tcgen05_wait_selftest(unsigned long long limit_ns, int* status, unsigned long long* waited_ns, cudaStream_t stream)
{
    if (limit_ns == 0 || limit_ns > 100000000ull) SPY_FAIL("wait self-test: the limit must lie between 1 ns and 100 ms, found %llu ns", limit_ns);
    wait_selftest_kernel<<<1, 32, 0, stream>>>(limit_ns, status, waited_ns);
    SPY_CHECK_LAUNCH("wait self-test");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// The same product for callers that cannot allocate device memory (declared in
// gemm_tcgen05_static.h; it has no counterpart in the reference).
//
// Some callers must not call cudaMalloc or anything that might: code that runs while a CUDA
// graph is being captured or inside a latency-critical serving loop where an allocation would
// synchronise the device, plug-ins loaded into a host process that owns all device memory and
// hands out none, and callers whose memory budget is fixed before the library is loaded.  For
// them the split-K scratch lives in the library image itself: a file-scope device array that
// every GPU which loads this library holds from load until the process exits.
//
// Limit: SPY_GEMM_STATIC_SCRATCH_FLOATS floats (16 MiB).  A product whose split-K plan needs
// more is refused with an error; it is not silently run another way.
//
// Set-up: the array's name is only a host-side handle; the device address comes from
// cudaGetSymbolAddress, asked once per device with that device current.  The first call on a
// device does this, so make that first call before any stream capture begins.
//
// Sharing: every call on a device uses the same array and leaves its partial sums there.
// Nothing has to be cleared between calls, because every element the reduction reads is
// written earlier in the same call.  Two calls that overlap on the GPU (different streams
// without an ordering between them) race on the array; order them.
#include "gemm_tcgen05_static.h"

static __device__ __align__(256) float g_gemm_static_scratch[SPY_GEMM_STATIC_SCRATCH_FLOATS];

extern "C" int spy_gemm_tcgen05_static_scratch(const void* A, long long lda, const void* W, long long ldw, void* C, int c_dtype, long long ldc,
                                               int M, int N, int K, int* status, cudaStream_t stream)
{
    constexpr int MAX_DEVICES = 64;
    static float* scratch_of_device[MAX_DEVICES] = {nullptr};
    if (M <= 0 || N <= 0) return 0;
    if (K <= 0 || K % 8 != 0) SPY_FAIL("gemm_tcgen05_static_scratch: K %d must be a positive multiple of 8", K);
    int splits;
    long long need;
    spy_gemm_tcgen05_plan(M, N, K, 0x7fffffffffffffffLL, &splits, &need);
    if (need > (long long)SPY_GEMM_STATIC_SCRATCH_FLOATS)
        SPY_FAIL("gemm_tcgen05_static_scratch: M=%d N=%d K=%d splits K %d ways and needs %lld floats of scratch; the built-in scratch holds %lld",
                 M, N, K, splits, need, (long long)SPY_GEMM_STATIC_SCRATCH_FLOATS);
    int device = -1;
    SPY_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= MAX_DEVICES) SPY_FAIL("gemm_tcgen05_static_scratch: device index %d is out of range", device);
    if (scratch_of_device[device] == nullptr) {
        float* ptr = nullptr;
        SPY_CUDA(cudaGetSymbolAddress((void**)&ptr, g_gemm_static_scratch));
        if (ptr == nullptr) SPY_FAIL("gemm_tcgen05_static_scratch: the built-in scratch has no address on device %d", device);
        scratch_of_device[device] = ptr;
    }
    return spy_gemm_tcgen05(A, lda, W, ldw, C, c_dtype, ldc, M, N, K, scratch_of_device[device], (long long)SPY_GEMM_STATIC_SCRATCH_FLOATS, status,
                            stream);
}
