// Weight gradient on the topology for token blocks, on the 5th-generation tensor cores.
//
// For every kept tile (r, c): dW[tile][i][j] = sum_t dy[t][16 r + i] * x[t][16 c + j]
// (`morph_stk::sdd_at_b`, morph/sparse/stk/backend/custom_ops.py:68-89).  Per tile that is a
// [16 x T] x [T x 16] product whose operands are as large as the tile's share of the activations,
// so computing kept tiles one by one is bound by re-reading dy and x.  This kernel computes whole
// 128 x 128 blocks of dW -- dy[:, 128 outputs]^T @ x[:, 128 inputs], a dense product over the token
// dimension -- and stores only the tiles the topology keeps (a block without a kept tile is never
// computed).  The token dimension of a block is split over several CTAs when the blocks alone do
// not fill the GPU; every split writes fp32 partial tiles and a second kernel adds them in split
// order (deterministic).
//
// One CTA = (block, split): warp 0 issues TMA loads of [64 tokens x 64 features] boxes (dy: two
// boxes for the 128 outputs, x: two for the 128 inputs; 128-byte swizzle) into a 4-stage ring,
// warp 1 issues tcgen05.mma (M = N = 128, K = 16 tokens, both operands M/N-major: a token is a
// 128-byte row of 64 features, so the activations are consumed as they lie in memory, without a
// transpose), warps 2..5 read the fp32 accumulators from tensor memory and store the kept tiles.
// Every mbarrier wait is bounded; on expiry the CTA records an error code and unwinds.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <mutex>
#include "common.h"
#include "tc_common.cuh"

namespace {

constexpr int kTok = 64;                       // tokens per pipeline stage
constexpr int kStages = 4;
constexpr int kBox = 64 * kTok * 2;            // one [64 tokens][64 features] bf16 box: 8 KB
constexpr int kStageBytes = 4 * kBox;          // dy (2 boxes) + x (2 boxes)
constexpr int kThreads = 192;
constexpr int kTmemCols = 128;
constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*align*/ + 64 * 4 /*tile map*/ + (2 * kStages + 1) * 8;

__device__ int g_sdd_error;                    // first error recorded by any CTA (0 = none)

struct SddParams {
    const int *blk_rc;        // [n_blocks][2] block row, block column (units of 128 features)
    const int *blk_tiles;     // [n_blocks][64] index of the kept tile at (tile row, tile col) of the block, or -1
    long long rows;           // tokens
    int tok_per_split;        // multiple of kTok
    float *dst;               // partial tiles [n_splits][nnz][256] (or the output itself for one split)
    long long split_stride;   // floats between splits
};

__global__ void __launch_bounds__(kThreads, 1)
sdd_blocks_kernel(const __grid_constant__ CUtensorMap tmap_dy, const __grid_constant__ CUtensorMap tmap_x,
                  const SddParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *stages = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    int *tiles_s = reinterpret_cast<int *>(stages + kStages * kStageBytes);
    uint64_t *full = reinterpret_cast<uint64_t *>(tiles_s + 64), *empty = full + kStages, *acc_full = empty + kStages;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x, split = blockIdx.y;
    const long long k_begin = (long long)split * p.tok_per_split;
    const long long k_end = min(p.rows, k_begin + p.tok_per_split);
    const int n_it = k_end > k_begin ? (int)((k_end - k_begin + kTok - 1) / kTok) : 0;

    if (threadIdx.x < 64) tiles_s[threadIdx.x] = p.blk_tiles[(long long)b * 64 + threadIdx.x];
    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kStages; ++s) { tc::mbar_init(tc::smem_u32(&full[s]), 1); tc::mbar_init(tc::smem_u32(&empty[s]), 1); }
        tc::mbar_init(tc::smem_u32(acc_full), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(tc::smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    volatile int *abort_flag = &abort_s;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        const int out0 = p.blk_rc[2 * b] * 128, in0 = p.blk_rc[2 * b + 1] * 128;
        for (int it = 0; it < n_it; ++it) {
            const int s = it % kStages;
            if (!tc::mbar_wait(tc::smem_u32(&empty[s]), ((it / kStages) & 1) ^ 1u, abort_flag, &g_sdd_error, 1)) break;
            if (lane == 0) {
                const uint32_t bar = tc::smem_u32(&full[s]);
                tc::mbar_arrive_expect_tx(bar, kStageBytes);
                const int tok = (int)(k_begin + (long long)it * kTok);
                const uint32_t dst = tc::smem_u32(stages + s * kStageBytes);
#pragma unroll
                for (int h = 0; h < 4; ++h) {
                    const CUtensorMap *map = h < 2 ? &tmap_dy : &tmap_x;
                    const int feat = (h < 2 ? out0 : in0) + (h & 1) * 64;
                    asm volatile(
                        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                        "[%0], [%1, {%2, %3}], [%4];\n"
                        ::"r"(dst + h * kBox), "l"(map), "r"(feat), "r"(tok), "r"(bar) : "memory");
                }
            }
            __syncwarp();
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        // instruction descriptor: D fp32 (bit 4), A and B bf16 (bits 7, 10), A and B M/N-major
        // (bits 15, 16), N >> 3 at bit 17, M >> 4 at bit 24
        constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (1u << 16) |
                                    ((128u >> 3) << 17) | ((128u >> 4) << 24);
        bool ok = true;
        for (int it = 0; it < n_it && ok; ++it) {
            const int s = it % kStages;
            ok = tc::mbar_wait(tc::smem_u32(&full[s]), (it / kStages) & 1, abort_flag, &g_sdd_error, 2);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (lane == 0) {
                const uint32_t a0 = tc::smem_u32(stages + s * kStageBytes), b0 = a0 + 2 * kBox;
#pragma unroll
                for (int kk = 0; kk < kTok / 16; ++kk) {
                    // M/N-major, 128-byte swizzle: a token is a 128-byte row of 64 features, 8 tokens
                    // are one 1024-byte atom (stride byte offset), the second half of the 128 features
                    // lies one box further (leading byte offset); 16 tokens per MMA = two atoms
                    const uint64_t ad = tc::make_smem_desc(a0 + kk * 2048, kBox, 1024, 2);
                    const uint64_t bd = tc::make_smem_desc(b0 + kk * 2048, kBox, 1024, 2);
                    tc::mma_f16(tmem, ad, bd, kIdesc, (it | kk) ? 1u : 0u);
                }
                tc::commit(tc::smem_u32(&empty[s]));
            }
            __syncwarp();
        }
        if (ok && lane == 0) {
            if (n_it > 0) tc::commit(tc::smem_u32(acc_full));
            else asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(tc::smem_u32(acc_full)) : "memory");
        }
        __syncwarp();
    } else {
        // ---------------- epilogue: warp w reads tensor-memory lanes 32 (w % 4) .. +31 ----------------
        const int q = warp & 3;
        if (tc::mbar_wait(tc::smem_u32(acc_full), 0, abort_flag, &g_sdd_error, 3, 1u << 26)) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int m = q * 32 + lane;                       // output feature of the block = accumulator lane
            const int tr = m >> 4;
            float *base = p.dst + (long long)split * p.split_stride + (m & 15) * 16;
#pragma unroll 1
            for (int tcol = 0; tcol < 8; ++tcol) {
                uint32_t r[16];
                if (n_it > 0) tc::ld16(tmem + ((uint32_t)(q * 32) << 16) + tcol * 16, r);
                else {
#pragma unroll
                    for (int i = 0; i < 16; ++i) r[i] = 0u;    // a split without tokens contributes zeros
                }
                const int idx = tiles_s[tr * 8 + tcol];
                if (idx >= 0) {
                    float4 *dst = reinterpret_cast<float4 *>(base + (long long)idx * 256);
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        dst[v] = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                             __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

// out[i] = sum over splits of part[s][i], in split order.
__global__ void sdd_reduce_kernel(const float *__restrict__ part, int n_splits, long long stride, long long n,
                                  float *__restrict__ out_f32, __nv_bfloat16 *__restrict__ out_bf16) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float v = part[i];
    for (int s = 1; s < n_splits; ++s) v += part[(long long)s * stride + i];
    if (out_f32) out_f32[i] = v;
    else out_bf16[i] = __float2bfloat16_rn(v);
}

std::mutex g_sdd_init_mutex;

}  // namespace

extern "C" int mortar_sdd_blocks(const void *dy, int64_t ld_dy, const void *x, int64_t ld_x, int64_t rows,
                                 int32_t out_features, int32_t in_features, const int32_t *blk_rc,
                                 const int32_t *blk_tiles, int32_t n_blocks, int32_t n_splits, int64_t nnz,
                                 float *scratch, int64_t scratch_floats, void *out, int32_t out_dtype,
                                 void *stream) {
    if (!dy || !x || !blk_rc || !blk_tiles || !out) return MORTAR_ERR_NULL;
    if (rows < 0 || out_features <= 0 || in_features <= 0 || n_blocks < 0 || n_splits < 1 || nnz < 0 ||
        ld_dy < out_features || ld_x < in_features || rows > 0x7fffffffLL)
        return MORTAR_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(dy) % 16) || (reinterpret_cast<uintptr_t>(x) % 16) || (ld_dy % 8) || (ld_x % 8) ||
        (reinterpret_cast<uintptr_t>(out) % 16) || (scratch && reinterpret_cast<uintptr_t>(scratch) % 16))
        return MORTAR_ERR_ALIGN;
    if (out_dtype != MORTAR_F32 && out_dtype != MORTAR_BF16) return MORTAR_ERR_DTYPE;
    if (n_blocks == 0 || nnz == 0) return MORTAR_OK;
    if (n_blocks > 0x7fffffff / 64 || n_splits > 65535) return MORTAR_ERR_CAPACITY;
    cudaStream_t st = (cudaStream_t)stream;
    const long long n_out = nnz * 256;
    if (rows == 0) {
        MORTAR_CUDA_CHECK(cudaMemsetAsync(out, 0, (size_t)n_out * (out_dtype == MORTAR_F32 ? 4 : 2), st));
        return MORTAR_OK;
    }
    // tokens per split: a multiple of the stage size; drop splits that would start past the end
    long long tps = ((rows + n_splits - 1) / n_splits + kTok - 1) / kTok * kTok;
    int splits = (int)((rows + tps - 1) / tps);
    const bool direct = splits == 1 && out_dtype == MORTAR_F32;
    if (!direct && (!scratch || scratch_floats < (long long)splits * n_out)) return MORTAR_ERR_CAPACITY;

    alignas(64) CUtensorMap map_dy, map_x;
    int rc = tc::encode_bf16_2d(&map_dy, dy, out_features, rows, ld_dy, 64, kTok);
    if (rc != MORTAR_OK) return rc;
    rc = tc::encode_bf16_2d(&map_x, x, in_features, rows, ld_x, 64, kTok);
    if (rc != MORTAR_OK) return rc;
    {
        static bool attr_set[64] = {false};
        int dev = 0;
        MORTAR_CUDA_CHECK(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64) return MORTAR_ERR_CAPACITY;
        std::lock_guard<std::mutex> lock(g_sdd_init_mutex);
        if (!attr_set[dev]) {
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(sdd_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
            attr_set[dev] = true;
        }
    }
    SddParams p;
    p.blk_rc = blk_rc; p.blk_tiles = blk_tiles; p.rows = rows; p.tok_per_split = (int)tps;
    p.dst = direct ? reinterpret_cast<float *>(out) : scratch;
    p.split_stride = n_out;
    sdd_blocks_kernel<<<dim3((unsigned)n_blocks, (unsigned)splits), kThreads, kSmemBytes, st>>>(map_dy, map_x, p);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    if (!direct) {
        sdd_reduce_kernel<<<(unsigned)((n_out + 255) / 256), 256, 0, st>>>(
            scratch, splits, n_out, n_out, out_dtype == MORTAR_F32 ? reinterpret_cast<float *>(out) : nullptr,
            out_dtype == MORTAR_BF16 ? reinterpret_cast<__nv_bfloat16 *>(out) : nullptr);
        MORTAR_CUDA_CHECK(cudaGetLastError());
    }
    return MORTAR_OK;
}

extern "C" int mortar_sdd_error(int32_t *code, int32_t reset) {
    if (!code) return MORTAR_ERR_NULL;
    int v = 0;
    MORTAR_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_sdd_error, sizeof(int)));
    *code = v;
    if (reset && v != 0) {
        const int zero = 0;
        MORTAR_CUDA_CHECK(cudaMemcpyToSymbol(g_sdd_error, &zero, sizeof(int)));
    }
    return MORTAR_OK;
}
