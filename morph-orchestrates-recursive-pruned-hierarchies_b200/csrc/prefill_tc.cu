// Prefill kernel: block-sparse ternary linear / SwiGLU over blocks of 128 activation rows on
// the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// One CTA owns 128 rows of the activation matrix and one panel of 16 weight tile rows, whose
// 256 fp32 accumulator columns live in tensor memory.  It walks the panel's non-empty chunks
// (64 input features each) through a 2-stage shared-memory ring:
//   warp 1        issues the TMA load of the [128 x 64] bf16 activation chunk (128-byte swizzle)
//   warps 2..5    expand the chunk's 2-bit tile codes into bf16 B tiles (K-major, no swizzle),
//                 stage the chunk's MMA run records, and later run the epilogue
//   warp 0        issues one tcgen05.mma per run (M=128, N=16*len, K=16) and commits
// The epilogue reads the accumulators with tcgen05.ld, applies the per-matrix scale, the
// reference's bf16 rounding points, SwiGLU and the cluster gates, and stores bf16 rows.
// Every mbarrier wait is bounded; on expiry the CTA records an error code and unwinds
// (tensor memory is released on every path).
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include "common.h"

namespace {

constexpr int kPanelRows = MORTAR_PANEL_ROWS;
constexpr int kChunkCols = MORTAR_CHUNK_COLS;
constexpr int kStages = 2;
constexpr int kRows = 128;                                   // activation rows per CTA (MMA M)
constexpr int kAStage = kRows * 128;                         // 16 KB
constexpr int kMaxTiles = kPanelRows * kChunkCols;           // 64 tiles per (panel, chunk)
constexpr int kBStage = kMaxTiles * 512;                     // 32 KB
constexpr int kRunStage = kMaxTiles * 16;                    // 1 KB
constexpr int kTmemCols = kPanelRows * 16;                   // 256
constexpr int kThreads = 192;
constexpr int kDecodeThreads = 128;
constexpr int kSmemBytes = kStages * (kAStage + kBStage + kRunStage) + 1024 /*align*/ + 128 /*barriers*/;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kMaxChunks = 1024;                             // in_features <= 65536

__device__ int g_prefill_error;   // first error recorded by any CTA (0 = none)

struct PrefillParams {
    const uint32_t *tiles;        // [n_tiles][16] words of canonical 2-bit codes
    const uint4 *runs;            // [n_runs]
    const int *cell_tile_ptr;     // [n_panels*n_chunks + 1]
    const int *cell_run_ptr;
    const uint32_t *panel_mask;   // [n_panels] rows that received at least one tile
    int n_chunks;
    int swiglu;
    int total_units;              // output tile rows (LINEAR) or hidden tile rows (SWIGLU)
    long long rows;
    __nv_bfloat16 *out;
    long long ld_out;
    float scale;                  // already rounded to bf16 when rounding is emulated
    const float *gates;
    long long ld_gates;
    int cluster_size;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false (after raising the CTA-wide abort flag and recording `code`)
// when the barrier did not complete within the limit or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          int code) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(&g_prefill_error, 0, code);
    return false;
}

__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo,
                                                   uint32_t layout) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}

__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ float rbf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// 16 stored 2-bit values (one tile row) -> 16 bf16 codes as two 16-byte vectors.
__device__ __forceinline__ void expand_row(uint32_t w, uint4 &lo, uint4 &hi) {
    const uint32_t k129 = 0x43014301u;
    uint32_t out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        uint32_t v = ((w >> (4 * i)) & 3u) | (((w >> (4 * i + 2)) & 3u) << 16) | 0x43004300u;
        __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162 *>(&v),
                                   *reinterpret_cast<const __nv_bfloat162 *>(&k129));
        out[i] = *reinterpret_cast<uint32_t *>(&r);
    }
    lo = make_uint4(out[0], out[1], out[2], out[3]);
    hi = make_uint4(out[4], out[5], out[6], out[7]);
}

__global__ void __launch_bounds__(kThreads, 2)
prefill_panel_kernel(const __grid_constant__ CUtensorMap tmap_x, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sA = smem;                                   // kStages x 16 KB, 1024-byte aligned
    uint8_t *sB = sA + kStages * kAStage;                 // kStages x 32 KB
    uint4 *sRuns = reinterpret_cast<uint4 *>(sB + kStages * kBStage);   // kStages x 64 records
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(sRuns) + kStages * kRunStage);
    // bars[0..1] full, bars[2..3] empty, bars[4] accumulators ready
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    __shared__ int tptr[kMaxChunks + 1], rptr[kMaxChunks + 1];   // this panel's cell pointers

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int panel = blockIdx.x;
    const long long row0 = (long long)blockIdx.y * kRows;
    for (int i = threadIdx.x; i <= p.n_chunks; i += kThreads) {
        tptr[i] = p.cell_tile_ptr[(long long)panel * p.n_chunks + i];
        rptr[i] = p.cell_run_ptr[(long long)panel * p.n_chunks + i];
    }

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kStages; ++s) {
            mbar_init(smem_u32(&bars[s]), kDecodeThreads + 1);
            mbar_init(smem_u32(&bars[kStages + s]), 1);
        }
        mbar_init(smem_u32(&bars[2 * kStages]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    volatile int *abort_flag = &abort_s;

    if (warp == 0) {
        // ---------------- MMA issue ----------------
        int it = 0;
        bool ok = true;
        for (int c = 0; c < p.n_chunks && ok; ++c) {
            const int r0 = rptr[c], r1 = rptr[c + 1];
            if (r1 == r0) continue;
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            ok = mbar_wait(smem_u32(&bars[s]), ph, abort_flag, 1);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (lane == 0) {
                const uint64_t a0 = make_smem_desc(smem_u32(sA + s * kAStage), 16, 1024, 2);
                const uint64_t b0 = make_smem_desc(smem_u32(sB + s * kBStage), 128, 256, 0);
                const uint4 *rr = sRuns + s * kMaxTiles;
                for (int r = 0; r < r1 - r0; ++r) {
                    const uint4 q = rr[r];
                    tc_mma(tmem + (q.z & 0xffffu), a0 + q.x, b0 + q.y, q.w, q.z >> 31);
                }
                tc_commit(smem_u32(&bars[kStages + s]));      // stage reusable once these MMAs retire
            }
            __syncwarp();
            ++it;
        }
        if (lane == 0) {
            if (ok && it > 0) tc_commit(smem_u32(&bars[2 * kStages]));
            else mbar_arrive(smem_u32(&bars[2 * kStages]));
        }
    } else if (warp == 1) {
        // ---------------- TMA producer ----------------
        int it = 0;
        for (int c = 0; c < p.n_chunks; ++c) {
            if (rptr[c + 1] == rptr[c]) continue;
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            if (!mbar_wait(smem_u32(&bars[kStages + s]), ph ^ 1u, abort_flag, 2)) break;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&bars[s]);
                mbar_arrive_expect_tx(bar, kAStage);
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                    "[%0], [%1, {%2, %3}], [%4];\n"
                    ::"r"(smem_u32(sA + s * kAStage)), "l"(&tmap_x), "r"(c * kChunkCols * 16),
                      "r"((int)row0), "r"(bar) : "memory");
            }
            __syncwarp();
            ++it;
        }
    } else {
        // ---------------- tile decode ----------------
        const int td = threadIdx.x - 64;
        int it = 0;
        bool ok = true;
        for (int c = 0; c < p.n_chunks && ok; ++c) {
            const int r0 = rptr[c], r1 = rptr[c + 1];
            if (r1 == r0) continue;
            const int t0 = tptr[c], t1 = tptr[c + 1];
            const int s = it % kStages;
            const uint32_t ph = (it / kStages) & 1;
            ok = mbar_wait(smem_u32(&bars[kStages + s]), ph ^ 1u, abort_flag, 3);
            if (!ok) break;
            if (td < r1 - r0) sRuns[s * kMaxTiles + td] = __ldg(p.runs + r0 + td);
            uint8_t *bdst = sB + s * kBStage;
            const int items = (t1 - t0) * 16;                  // (tile, row) pairs
            for (int item = td; item < items; item += kDecodeThreads) {
                const int tile = item >> 4, row = item & 15;
                const uint32_t w = __ldg(p.tiles + (long long)(t0 + tile) * 16 + row);
                uint4 lo, hi;
                expand_row(w, lo, hi);
                uint8_t *d = bdst + tile * 512 + (row >> 3) * 256 + (row & 7) * 16;
                *reinterpret_cast<uint4 *>(d) = lo;            // features 0..7 of the tile column
                *reinterpret_cast<uint4 *>(d + 128) = hi;      // features 8..15
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            mbar_arrive(smem_u32(&bars[s]));
            ++it;
        }
        // ---------------- epilogue ----------------
        if (ok) ok = mbar_wait(smem_u32(&bars[2 * kStages]), 0, abort_flag, 4);
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const int q = warp & 3;                            // tensor-memory lane quadrant of this warp
            const long long row = row0 + q * 32 + lane;
            const bool in_range = row < p.rows;
            const uint32_t taddr = tmem + ((uint32_t)(q * 32) << 16);
            const uint32_t mask = p.panel_mask[panel];
            const int units = p.swiglu ? kPanelRows / 2 : kPanelRows;
            for (int j = 0; j < units; ++j) {
                uint32_t a[16], b[16];
                tc_ld16(taddr + j * 16, a);
                if (p.swiglu) tc_ld16(taddr + (units + j) * 16, b);
                const bool live_a = (mask >> j) & 1u;
                const bool live_b = p.swiglu ? ((mask >> (units + j)) & 1u) : true;
                const long long col0 = ((long long)panel * units + j) * 16;
                uint32_t packed[8];
#pragma unroll
                for (int e = 0; e < 16; e += 2) {
                    float v[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        float g = live_a ? rbf(p.scale * __uint_as_float(a[e + h])) : 0.f;
                        if (p.swiglu) {
                            const float u = live_b ? rbf(p.scale * __uint_as_float(b[e + h])) : 0.f;
                            const float sg = rbf(g / (1.f + expf(-g)));
                            float hv = rbf(sg * u);
                            if (p.gates != nullptr && in_range) {
                                const float gt = p.gates[row * p.ld_gates + (col0 + e + h) / p.cluster_size];
                                hv = gt > 0.f ? rbf(hv * rbf(gt)) : 0.f;
                            }
                            g = hv;
                        }
                        v[h] = g;
                    }
                    __nv_bfloat162 pr = __floats2bfloat162_rn(v[0], v[1]);
                    packed[e >> 1] = *reinterpret_cast<uint32_t *>(&pr);
                }
                if (in_range && panel * units + j < p.total_units) {
                    uint4 *dst = reinterpret_cast<uint4 *>(p.out + row * p.ld_out + col0);
                    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

int get_encode_fn(EncodeTiledFn *out) {
    static EncodeTiledFn cached = nullptr;
    if (!cached) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        MORTAR_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) {
            mortar_set_cuda_error("cudaGetDriverEntryPoint", "cuTensorMapEncodeTiled unavailable");
            return MORTAR_ERR_CUDA;
        }
        cached = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = cached;
    return MORTAR_OK;
}

inline bool aligned_to(const void *ptr, size_t a) { return (reinterpret_cast<uintptr_t>(ptr) % a) == 0; }

}  // namespace

extern "C" int mortar_linear_tc(const mortar_sched *w, const void *x, int64_t ldx, int64_t rows,
                                void *out, int64_t ld_out, const float *gates, int64_t ld_gates,
                                int32_t cluster_size, void *stream) {
    if (!w || !x || !out || !w->cell_tile_ptr || !w->cell_run_ptr || !w->panel_mask) return MORTAR_ERR_NULL;
    if (w->n_tiles > 0 && (!w->tiles || !w->runs)) return MORTAR_ERR_NULL;
    if (w->tile_rows <= 0 || w->tile_cols <= 0 || rows < 0) return MORTAR_ERR_SHAPE;
    const int K = w->tile_cols * 16;
    const int units = w->swiglu ? w->tile_rows / 2 : w->tile_rows;
    if (ldx < K || ld_out < (int64_t)units * 16) return MORTAR_ERR_SHAPE;
    if (!aligned_to(x, 16) || (ldx % 8) || !aligned_to(out, 16) || (ld_out % 8)) return MORTAR_ERR_ALIGN;
    if (gates && (cluster_size <= 0 || !w->swiglu)) return MORTAR_ERR_SHAPE;
    if (w->n_chunks > kMaxChunks) return MORTAR_ERR_CAPACITY;
    if (rows == 0) return MORTAR_OK;
    const int64_t row_blocks = (rows + kRows - 1) / kRows;
    if (row_blocks > 65535) return MORTAR_ERR_CAPACITY;

    EncodeTiledFn encode;
    int rc = get_encode_fn(&encode);
    if (rc != MORTAR_OK) return rc;
    alignas(64) CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)ldx * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)kRows};
    const cuuint32_t estride[2] = {1, 1};
    CUresult cr = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x), gdim, gstride,
                         box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        mortar_set_cuda_error("cuTensorMapEncodeTiled", "failed to encode the activation tensor map");
        return MORTAR_ERR_CUDA;
    }

    static bool attr_set = false;
    if (!attr_set) {
        MORTAR_CUDA_CHECK(cudaFuncSetAttribute(prefill_panel_kernel,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
        attr_set = true;
    }
    PrefillParams p;
    p.tiles = reinterpret_cast<const uint32_t *>(w->tiles);
    p.runs = reinterpret_cast<const uint4 *>(w->runs);
    p.cell_tile_ptr = w->cell_tile_ptr;
    p.cell_run_ptr = w->cell_run_ptr;
    p.panel_mask = w->panel_mask;
    p.n_chunks = w->n_chunks;
    p.swiglu = w->swiglu;
    p.total_units = units;
    p.rows = rows;
    p.out = reinterpret_cast<__nv_bfloat16 *>(out);
    p.ld_out = ld_out;
    p.scale = __bfloat162float(__float2bfloat16_rn(w->scale));
    p.gates = gates;
    p.ld_gates = ld_gates;
    p.cluster_size = cluster_size > 0 ? cluster_size : 1;
    dim3 grid((unsigned)w->n_panels, (unsigned)row_blocks);
    prefill_panel_kernel<<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(tmap, p);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

extern "C" int mortar_mlp_prefill(const mortar_sched *gate_up, const mortar_sched *down, const void *x,
                                  int64_t ldx, int64_t rows, const float *gates, int64_t ld_gates,
                                  int32_t n_clusters, void *y, int64_t ldy, void *workspace,
                                  int64_t workspace_bytes, void *stream) {
    if (!gate_up || !down || !x || !y || !workspace) return MORTAR_ERR_NULL;
    if (!gate_up->swiglu || down->swiglu) return MORTAR_ERR_SHAPE;
    const int d_model = gate_up->tile_cols * 16, d_ff = gate_up->tile_rows * 8;
    if (down->tile_cols * 16 != d_ff || down->tile_rows * 16 != d_model) return MORTAR_ERR_SHAPE;
    if (gates && (n_clusters <= 0 || d_ff % n_clusters)) return MORTAR_ERR_SHAPE;
    if (!aligned_to(workspace, 256)) return MORTAR_ERR_ALIGN;
    if (workspace_bytes < rows * (int64_t)d_ff * 2) return MORTAR_ERR_CAPACITY;
    int rc = mortar_linear_tc(gate_up, x, ldx, rows, workspace, d_ff, gates, ld_gates,
                              gates ? d_ff / n_clusters : 0, stream);
    if (rc != MORTAR_OK) return rc;
    return mortar_linear_tc(down, workspace, d_ff, rows, y, ldy, nullptr, 0, 0, stream);
}

extern "C" int mortar_prefill_error(int32_t *code, int32_t reset) {
    if (!code) return MORTAR_ERR_NULL;
    int v = 0;
    MORTAR_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_prefill_error, sizeof(int)));
    *code = v;
    if (reset && v != 0) {
        const int zero = 0;
        MORTAR_CUDA_CHECK(cudaMemcpyToSymbol(g_prefill_error, &zero, sizeof(int)));
    }
    return MORTAR_OK;
}
