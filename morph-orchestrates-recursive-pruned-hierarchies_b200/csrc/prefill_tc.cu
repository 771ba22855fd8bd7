// Prefill kernel: block-sparse ternary linear / SwiGLU over blocks of 128 activation rows on
// the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// One CTA owns 128 rows of the activation matrix and one panel of 16 weight tile rows, whose
// 256 fp32 accumulator columns live in tensor memory.  It walks the panel's schedule steps
// (each: one 64-feature activation chunk and up to 48 weight tiles) through two rings:
//   warp 1        issues the TMA loads of the [128 x 64] bf16 activation chunks (128-byte
//                 swizzle) into a 3-stage ring, ahead of their use
//   warps 2..5    expand each step's 2-bit tile codes into bf16 B tiles (K-major, no swizzle)
//                 in a 2-stage ring, stage the step's MMA run records, and later run the
//                 epilogue; code words of the next step are fetched before the current one
//                 is expanded
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
constexpr int kAStages = 3;                                  // activation-chunk ring
constexpr int kBStages = 2;                                  // expanded-tile ring
constexpr int kRows = 128;                                   // activation rows per CTA (MMA M)
constexpr int kAStage = kRows * 128;                         // 16 KB
constexpr int kStepTiles = MORTAR_STEP_TILES;                // tiles per step
constexpr int kBStage = kStepTiles * 512;                    // 24 KB
constexpr int kRunStage = kStepTiles * 16;                   // run records of one step
constexpr int kTmemCols = kPanelRows * 16;                   // 256
constexpr int kThreads = 192;
constexpr int kDecodeThreads = 128;
constexpr int kWordsPerThread = kStepTiles * 16 / kDecodeThreads;   // code words a decoder expands per step
constexpr int kSmemBytes = kAStages * kAStage + kBStages * (kBStage + kRunStage) + 1024 /*align*/ + 128 /*barriers*/;
constexpr uint32_t kWaitLimit = 1u << 22;
constexpr int kMaxSteps = 512;                               // steps of one panel held in shared memory

__device__ int g_prefill_error;   // first error recorded by any CTA (0 = none)

struct PrefillParams {
    const uint32_t *tiles;        // [n_tiles][16] words of canonical 2-bit codes
    const uint4 *runs;            // [n_runs]
    const int *panel_step_ptr;    // [n_panels + 1]
    const int *step_tile_ptr;     // [n_steps + 1]
    const int *step_run_ptr;      // [n_steps + 1]
    const uint32_t *step_chunk;   // [n_steps] chunk | reuse<<30 | last<<31
    const uint32_t *panel_mask;   // [n_panels] rows that received at least one tile
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

// Descriptors are passed as (low, high) words: only the low word (start address) changes
// between MMAs of a step, so the issuing lane does 32-bit adds only.
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                       uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 da, db;\n"
        "setp.ne.b32 p, %6, 0;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate));
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
    uint8_t *sA = smem;                                   // kAStages x 16 KB, 1024-byte aligned
    uint8_t *sB = sA + kAStages * kAStage;                // kBStages x 24 KB
    uint4 *sRuns = reinterpret_cast<uint4 *>(sB + kBStages * kBStage);
    uint64_t *bars = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(sRuns) + kBStages * kRunStage);
    uint64_t *a_full = bars, *a_empty = bars + kAStages;
    uint64_t *b_full = bars + 2 * kAStages, *b_empty = b_full + kBStages;
    uint64_t *acc_full = b_empty + kBStages;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    __shared__ int s_tile[kMaxSteps + 1], s_run[kMaxSteps + 1];   // this panel's step pointers
    __shared__ uint32_t s_chunk[kMaxSteps];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int panel = blockIdx.x;
    const long long row0 = (long long)blockIdx.y * kRows;
    const int step0 = p.panel_step_ptr[panel];
    const int n_steps = p.panel_step_ptr[panel + 1] - step0;
    for (int i = threadIdx.x; i <= n_steps; i += kThreads) {
        s_tile[i] = p.step_tile_ptr[step0 + i];
        s_run[i] = p.step_run_ptr[step0 + i];
        if (i < n_steps) s_chunk[i] = p.step_chunk[step0 + i];
    }

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kAStages; ++s) {
            mbar_init(smem_u32(&a_full[s]), 1);
            mbar_init(smem_u32(&a_empty[s]), 1);
        }
        for (int s = 0; s < kBStages; ++s) {
            mbar_init(smem_u32(&b_full[s]), kDecodeThreads);
            mbar_init(smem_u32(&b_empty[s]), 1);
        }
        mbar_init(smem_u32(acc_full), 1);
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
        int a_it = -1;                                     // activation chunks consumed so far - 1
        bool ok = true;
        for (int i = 0; i < n_steps && ok; ++i) {
            const uint32_t ck = s_chunk[i];
            const int bs = i % kBStages;
            if (!(ck & 0x40000000u)) {                     // this step starts a new activation chunk
                ++a_it;
                ok = mbar_wait(smem_u32(&a_full[a_it % kAStages]), (a_it / kAStages) & 1, abort_flag, 1);
                if (!ok) break;
            }
            ok = mbar_wait(smem_u32(&b_full[bs]), (i / kBStages) & 1, abort_flag, 5);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            if (lane == 0) {
                const int as = a_it % kAStages;
                const uint64_t a0 = make_smem_desc(smem_u32(sA + as * kAStage), 16, 1024, 2);
                const uint64_t b0 = make_smem_desc(smem_u32(sB + bs * kBStage), 128, 256, 0);
                const uint32_t a_lo = (uint32_t)a0, a_hi = (uint32_t)(a0 >> 32);
                const uint32_t b_lo = (uint32_t)b0, b_hi = (uint32_t)(b0 >> 32);
                const uint4 *rr = sRuns + bs * kStepTiles;
                const int nrun = s_run[i + 1] - s_run[i];
                for (int r = 0; r < nrun; r += 4) {
                    // fetch four run records, then issue: the loads do not wait behind the MMAs
                    uint4 q[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) q[k] = rr[min(r + k, nrun - 1)];
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        if (r + k < nrun)
                            tc_mma(tmem + (q[k].z & 0xffffu), a_lo + q[k].x, a_hi, b_lo + q[k].y, b_hi,
                                   q[k].w, q[k].z >> 31);
                }
                tc_commit(smem_u32(&b_empty[bs]));         // B stage reusable once these MMAs retire
                if (ck & 0x80000000u) tc_commit(smem_u32(&a_empty[as]));   // last step on this chunk
            }
            __syncwarp();
        }
        if (lane == 0) {
            if (ok && n_steps > 0) tc_commit(smem_u32(acc_full));
            else mbar_arrive(smem_u32(acc_full));
        }
    } else if (warp == 1) {
        // ---------------- TMA producer ----------------
        int a_it = 0;
        for (int i = 0; i < n_steps; ++i) {
            const uint32_t ck = s_chunk[i];
            if (ck & 0x40000000u) continue;
            const int as = a_it % kAStages;
            if (!mbar_wait(smem_u32(&a_empty[as]), ((a_it / kAStages) & 1) ^ 1u, abort_flag, 2)) break;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&a_full[as]);
                mbar_arrive_expect_tx(bar, kAStage);
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                    "[%0], [%1, {%2, %3}], [%4];\n"
                    ::"r"(smem_u32(sA + as * kAStage)), "l"(&tmap_x),
                      "r"((int)(ck & 0xffffffu) * kChunkCols * 16), "r"((int)row0), "r"(bar) : "memory");
            }
            __syncwarp();
            ++a_it;
        }
    } else {
        // ---------------- tile decode ----------------
        const int td = threadIdx.x - 64;
        bool ok = true;
        uint32_t cur[kWordsPerThread], nxt[kWordsPerThread];
        uint4 cur_run = make_uint4(0, 0, 0, 0), nxt_run = make_uint4(0, 0, 0, 0);
        auto fetch = [&](int i, uint32_t (&w)[kWordsPerThread], uint4 &run) {
            const int t0 = s_tile[i], items = (s_tile[i + 1] - t0) * 16;
#pragma unroll
            for (int k = 0; k < kWordsPerThread; ++k) {
                const int item = td + k * kDecodeThreads;
                w[k] = item < items ? __ldg(p.tiles + (long long)t0 * 16 + item) : 0u;
            }
            if (td < s_run[i + 1] - s_run[i]) run = __ldg(p.runs + s_run[i] + td);
        };
        if (n_steps > 0) fetch(0, cur, cur_run);
        for (int i = 0; i < n_steps && ok; ++i) {
            if (i + 1 < n_steps) fetch(i + 1, nxt, nxt_run);
            const int bs = i % kBStages;
            ok = mbar_wait(smem_u32(&b_empty[bs]), ((i / kBStages) & 1) ^ 1u, abort_flag, 3);
            if (!ok) break;
            if (td < s_run[i + 1] - s_run[i]) sRuns[bs * kStepTiles + td] = cur_run;
            uint8_t *bdst = sB + bs * kBStage;
            const int items = (s_tile[i + 1] - s_tile[i]) * 16;        // (tile, row) pairs
#pragma unroll
            for (int k = 0; k < kWordsPerThread; ++k) {
                const int item = td + k * kDecodeThreads;
                if (item < items) {
                    const int tile = item >> 4, row = item & 15;
                    uint4 lo, hi;
                    expand_row(cur[k], lo, hi);
                    uint8_t *d = bdst + tile * 512 + (row >> 3) * 256 + (row & 7) * 16;
                    *reinterpret_cast<uint4 *>(d) = lo;        // features 0..7 of the tile column
                    *reinterpret_cast<uint4 *>(d + 128) = hi;  // features 8..15
                }
            }
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            mbar_arrive(smem_u32(&b_full[bs]));
#pragma unroll
            for (int k = 0; k < kWordsPerThread; ++k) cur[k] = nxt[k];
            cur_run = nxt_run;
        }
        // ---------------- epilogue ----------------
        if (ok) ok = mbar_wait(smem_u32(acc_full), 0, abort_flag, 4);
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
    if (!w || !x || !out || !w->panel_step_ptr || !w->step_tile_ptr || !w->step_run_ptr ||
        !w->step_chunk || !w->panel_mask)
        return MORTAR_ERR_NULL;
    if (w->n_tiles > 0 && (!w->tiles || !w->runs)) return MORTAR_ERR_NULL;
    if (w->tile_rows <= 0 || w->tile_cols <= 0 || rows < 0) return MORTAR_ERR_SHAPE;
    const int K = w->tile_cols * 16;
    const int units = w->swiglu ? w->tile_rows / 2 : w->tile_rows;
    if (ldx < K || ld_out < (int64_t)units * 16) return MORTAR_ERR_SHAPE;
    if (!aligned_to(x, 16) || (ldx % 8) || !aligned_to(out, 16) || (ld_out % 8)) return MORTAR_ERR_ALIGN;
    if (gates && (cluster_size <= 0 || !w->swiglu)) return MORTAR_ERR_SHAPE;
    if (w->max_panel_steps > kMaxSteps) return MORTAR_ERR_CAPACITY;
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
    p.panel_step_ptr = w->panel_step_ptr;
    p.step_tile_ptr = w->step_tile_ptr;
    p.step_run_ptr = w->step_run_ptr;
    p.step_chunk = w->step_chunk;
    p.panel_mask = w->panel_mask;
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
