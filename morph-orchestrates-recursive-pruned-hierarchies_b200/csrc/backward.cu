// Weight gradient of the carved linear on its topology: for every kept 16x16 tile (r, c)
//     dW[tile][i][j] = sum_t dy[t][16 r + i] * x[t][16 c + j]
// the sampled product the reference computes with stk `sdd` as `stk_sdd_at_b`
// (morph/sparse/stk/backend/custom_ops.py:68-89, triton_kernels.py:43-78, 357-411): bf16 operands,
// fp32 accumulation.  (The input gradient needs no kernel of its own: dx = dy @ W is the forward
// kernel on the transposed matrix.)
//
// One CTA = up to 8 kept tiles of one tile row (one warp per tile).  The token dimension is the
// MMA's K: per chunk of 64 tokens the CTA stages the 16 dy columns of its tile row once and the 16
// x columns of each of its tiles, then every warp reads its A fragments (dy^T, shared by all
// warps) and B fragments (its own x tile) with transposing matrix loads and issues
// mma.m16n8k16.  This is a functional training-side operator, not a tuned one: the activations
// are re-read once per group of 8 tiles.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "common.h"

namespace {

constexpr int kTilesPerCta = 8;
constexpr int kChunk = 64;                 // tokens staged per step

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// grid.x = work items; item -> (tile row, first tile of the row's list, count <= 8) through
// item_ptr (prefix over tile rows of ceil(nnz_row / 8)).
__global__ void __launch_bounds__(kTilesPerCta * 32)
sdd_tiles_kernel(const __nv_bfloat16 *__restrict__ dy, long long ld_dy, const __nv_bfloat16 *__restrict__ x,
                 long long ld_x, long long rows, const int *__restrict__ row_ptr,
                 const unsigned short *__restrict__ col_idx, const int *__restrict__ item_row,
                 const int *__restrict__ item_first, float *__restrict__ out_f32,
                 __nv_bfloat16 *__restrict__ out_bf16) {
    // token-major staging: [token][16 columns] bf16 = 32 bytes per token row; 16-byte units are
    // XOR-swizzled by (token >> 2) & 1 so the 8 rows of a transposed 8x8 load fall in distinct banks
    __shared__ __align__(16) __nv_bfloat16 s_dy[kChunk][16];
    __shared__ __align__(16) __nv_bfloat16 s_x[kTilesPerCta][kChunk][16];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int trow = item_row[blockIdx.x];
    const int first = item_first[blockIdx.x];
    const int n_tiles = min(kTilesPerCta, row_ptr[trow + 1] - first);
    const bool have = warp < n_tiles;
    const int tcol = have ? (int)col_idx[first + warp] : 0;
    float acc[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};

    for (long long t0 = 0; t0 < rows; t0 += kChunk) {
        // stage: 64 tokens x 16 columns = 128 16-byte pieces per operand tile
        for (int e = threadIdx.x; e < kChunk * 2; e += blockDim.x) {
            const int tk = e >> 1, half = e & 1;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (t0 + tk < rows) v = *reinterpret_cast<const uint4 *>(dy + (t0 + tk) * ld_dy + trow * 16 + half * 8);
            *reinterpret_cast<uint4 *>(&s_dy[tk][(half ^ ((tk >> 2) & 1)) * 8]) = v;
        }
        if (have) {
            for (int e = lane; e < kChunk * 2; e += 32) {
                const int tk = e >> 1, half = e & 1;
                uint4 v = make_uint4(0, 0, 0, 0);
                if (t0 + tk < rows) v = *reinterpret_cast<const uint4 *>(x + (t0 + tk) * ld_x + tcol * 16 + half * 8);
                *reinterpret_cast<uint4 *>(&s_x[warp][tk][(half ^ ((tk >> 2) & 1)) * 8]) = v;
            }
        }
        __syncthreads();
        if (have) {
#pragma unroll
            for (int k0 = 0; k0 < kChunk; k0 += 16) {
                // A = dy^T [16 features x 16 tokens]: four 8x8 blocks (feature half, token half);
                // stored token-major, so a transposing load of rows (token, 8 features) yields
                // the row-major A fragment.  Lane l supplies the row address of matrix l>>3:
                // matrices 0..3 = (f 0-7, t 0-7), (f 8-15, t 0-7), (f 0-7, t 8-15), (f 8-15, t 8-15)
                const int m = lane >> 3, r = lane & 7;
                const int tk = k0 + (m >> 1) * 8 + r, fh = m & 1;
                uint32_t a0, a1, a2, a3;
                ldmatrix_x4_trans(smem_u32(&s_dy[tk][(fh ^ ((tk >> 2) & 1)) * 8]), a0, a1, a2, a3);
                // B = x [16 tokens x 16 columns] as two n8 halves; the B fragment wants (k pair, n)
                // = rows of tokens: matrices 0..3 = (t 0-7, c 0-7), (t 8-15, c 0-7), (t 0-7, c 8-15),
                // (t 8-15, c 8-15); stored token-major, a transposing load gives k-pairs per column
                const int tkb = k0 + (m & 1) * 8 + r, ch = m >> 1;
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4_trans(smem_u32(&s_x[warp][tkb][(ch ^ ((tkb >> 2) & 1)) * 8]), b0, b1, b2, b3);
                mma_16816(acc[0], a0, a1, a2, a3, b0, b1);
                mma_16816(acc[1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();
    }
    if (!have) return;
    // acc[h][0..3] = (feature g, column 8h + 2t), (g, 8h + 2t + 1), (g + 8, 8h + 2t), (g + 8, 8h + 2t + 1)
    const int g = lane >> 2, t = lane & 3;
    const long long base = (long long)(first + warp) * 256;
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int fi = g + 8 * (i >> 1), cj = 8 * h + 2 * t + (i & 1);
            if (out_f32 != nullptr) out_f32[base + fi * 16 + cj] = acc[h][i];
            else out_bf16[base + fi * 16 + cj] = __float2bfloat16_rn(acc[h][i]);
        }
}

}  // namespace

extern "C" int mortar_sdd_tiles(const void *dy, int64_t ld_dy, const void *x, int64_t ld_x, int64_t rows,
                                const int32_t *row_ptr, const uint16_t *col_idx, int32_t tile_rows,
                                int32_t tile_cols, const int32_t *item_row, const int32_t *item_first,
                                int32_t n_items, void *out, int32_t out_dtype, void *stream) {
    if (!dy || !x || !row_ptr || !col_idx || !item_row || !item_first || !out) return MORTAR_ERR_NULL;
    if (rows < 0 || tile_rows <= 0 || tile_cols <= 0 || n_items < 0) return MORTAR_ERR_SHAPE;
    if (ld_dy < (int64_t)tile_rows * 16 || ld_x < (int64_t)tile_cols * 16) return MORTAR_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(dy) % 16) || (reinterpret_cast<uintptr_t>(x) % 16) || (ld_dy % 8) || (ld_x % 8))
        return MORTAR_ERR_ALIGN;
    if (out_dtype != MORTAR_F32 && out_dtype != MORTAR_BF16) return MORTAR_ERR_DTYPE;
    if (n_items == 0) return MORTAR_OK;
    sdd_tiles_kernel<<<(unsigned)n_items, kTilesPerCta * 32, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const __nv_bfloat16 *>(dy), ld_dy, reinterpret_cast<const __nv_bfloat16 *>(x), ld_x, rows,
        row_ptr, col_idx, item_row, item_first, out_dtype == MORTAR_F32 ? reinterpret_cast<float *>(out) : nullptr,
        out_dtype == MORTAR_BF16 ? reinterpret_cast<__nv_bfloat16 *>(out) : nullptr);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}
