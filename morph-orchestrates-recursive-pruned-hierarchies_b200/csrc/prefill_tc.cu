// Prefill kernel: block-sparse ternary linear / SwiGLU over blocks of 128 activation rows on
// the 5th-generation tensor cores (tcgen05.mma, accumulators in tensor memory).
//
// Persistent: one CTA per SM loops over work items.  An item is 128 activation rows x a PAIR
// of panels (2 x 16 weight tile rows); each panel has its own pipeline ("pipe") and its own
// 256 fp32 accumulator columns in tensor memory, and both pipes consume the same stream of
// activation chunks, so an activation chunk is fetched once for 32 tile rows.
// Warp roles (20 warps; a warp's scheduler is its index modulo 4, so the three single-lane
// issuing roles sit together on scheduler 3, away from the arithmetic of the decode warps):
//   warps 0..7    epilogue (4 per pipe, one per tensor-memory lane quadrant): tcgen05.ld,
//                 per-matrix scale, the reference's bf16 rounding points, SwiGLU, cluster gates,
//                 bf16 stores; idle while the MMAs of an item run
//   warps 11, 15  MMA issue, one per pipe: one tcgen05.mma per run (M=128, N=16*len, K=16) from
//                 16-bit run records, tcgen05.commit to hand stages back
//   warp 19       TMA producer: per activation chunk one tiled [128 x 64] bf16 load (128-byte
//                 swizzle) into a 4-stage ring
//   warps 8, 9, 10, 12 (pipe 0) and 13, 14, 16, 17 (pipe 1)   decode: read the step records
//                 (run list + packed 2-bit codes) straight from global memory one step ahead
//                 and expand the codes into bf16 B tiles (K-major, no swizzle) in a 3-stage ring
//   warp 18       unused
// Every mbarrier wait is bounded; on expiry the CTA records an error code, every role unwinds
// and tensor memory is released.
#include <cuda.h>
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <atomic>
#include <mutex>
#include <type_traits>
#include "common.h"
#include "decode.cuh"

namespace {

constexpr int kPanelRows = MORTAR_PANEL_ROWS;
constexpr int kChunkCols = MORTAR_CHUNK_COLS;
constexpr int kStepTiles = MORTAR_STEP_TILES;                // 48 tile slots per step
constexpr int kPipes = 2;                                    // panels executed side by side per item
constexpr int kAStages = 4;                                  // activation-chunk ring (shared)
constexpr int kBStages = 3;                                  // expanded-tile ring, per pipe
constexpr int kRows = 128;                                   // activation rows per item (MMA M)
constexpr int kAStage = kRows * 128;                         // 16 KB
constexpr int kBTiles = kStepTiles * 512;                    // 24 KB of expanded tiles
constexpr int kRunBytes = 128;                               // the step's 16-bit run records (up to 48)
constexpr int kBStage = kBTiles + kRunBytes + 128;           // + the step header; pitch stays a multiple of 128
constexpr int kAccCols = kPanelRows * 16;                    // 256 accumulator columns per pipe
constexpr int kTmemCols = kPipes * kAccCols;                 // 512
constexpr int kDecodeThreads = 128;                          // per pipe
constexpr int kEpilogueWarps = 4 * kPipes;
constexpr int kEpilogueThreads = 32 * kEpilogueWarps;
constexpr int kMmaWarp0 = 11, kMmaWarp1 = 15, kTmaWarp = 19, kIdleWarp = 18;
constexpr int kThreads = 32 * 20;                            // 640
constexpr int kWordsPerThread = kStepTiles * 16 / kDecodeThreads;   // 6 row words per decoder per step
constexpr int kStepSlotsI8 = MORTAR_STEP_SLOTS_I8;                  // int8 schedule: 24 slots of 16 x 32 codes
constexpr int kRowsPerThreadI8 = kStepSlotsI8 * 16 / kDecodeThreads; // 3 row records (16 bytes) per decoder per step
constexpr int kNumBars = 2 * kAStages + kPipes * 2 * kBStages + 2;
constexpr int kSmemBytes = kAStages * kAStage + kPipes * kBStages * kBStage + kNumBars * 8 + 1024 /*align*/;
constexpr uint32_t kWaitLimit = 1u << 22;
static_assert(kStepTiles * 2 <= kRunBytes, "run records do not fit their area");
static_assert(kSmemBytes <= 227 * 1024, "shared memory budget");

__device__ int g_prefill_error;   // first error recorded by any CTA (0 = none)

// Per-role cycle accounting for profiling builds (-DMORTAR_PREFILL_TIMING): every role of pipe 0
// sums the cycles it spends in each of its phases; CTA 0 adds them to g_prefill_ticks.
#ifdef MORTAR_PREFILL_TIMING
__device__ unsigned long long g_prefill_ticks[40];
#define PF_DECL long long tk[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long tprev = clock64()
#define PF_ACC(i) do { const long long tn_ = clock64(); tk[i] += tn_ - tprev; tprev = tn_; } while (0)
#define PF_PUT(base, cond) do { if ((cond) && blockIdx.x == 0) for (int i_ = 0; i_ < 8; ++i_) \
        atomicAdd(&g_prefill_ticks[(base) + i_], (unsigned long long)tk[i_]); } while (0)
#else
#define PF_DECL
#define PF_ACC(i)
#define PF_PUT(base, cond)
#endif

struct PrefillParams {
    const uint8_t *step_data;     // step records
    const uint32_t *step_off;     // [n_steps + 1], 16-byte units
    const uint32_t *step_meta;    // [n_steps] chunk | reuse<<30 | last<<31
    const int *panel_step_ptr;    // [n_panels + 1]
    const uint32_t *panel_mask;   // [n_panels] rows that received at least one tile
    int n_panels;
    int n_items;                  // n_panels * row blocks
    int swiglu;
    int total_units;              // output tile rows (LINEAR) or hidden tile rows (SWIGLU)
    long long rows;
    __nv_bfloat16 *out;
    long long ld_out;
    float scale;                  // per-matrix scale rounded to bf16
    const float *x_scale;         // int8 arm: per-row activation scales [rows]
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

// Same, for roles that run ahead of the critical path: backs off between polls so the
// spinning warp does not take issue slots from the warps doing work.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                                  int code) {
    for (uint32_t i = 0; i < kWaitLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        __nanosleep(64);
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
// The same with the accumulate flag fixed at compile time (no predicate to compute per instruction).
template <bool ACC>
__device__ __forceinline__ void tc_mma_lit(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                           uint32_t b_hi, uint32_t idesc) {
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 da, db;\n"
        "setp.eq.u32 p, %6, 1;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %5, p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "n"(ACC ? 1 : 0));
}
// One stage of a step: the poll of the NEXT stage's barrier and this stage's four MMAs (16 features
// each, descriptor addresses 2 units apart) as one instruction sequence, so that the poll's result
// is first read after the MMAs have issued and its latency runs under them.  PAIR selects
// cta_group::2.  Returns whether the polled phase had completed.
template <bool FIRST_ACC, bool PAIR>
__device__ __forceinline__ bool tc_poll_mma4(uint32_t next_bar, uint32_t next_parity, uint32_t d_tmem, uint32_t a_lo,
                                             uint32_t b_lo, uint32_t d_hi, uint32_t idesc) {
    uint32_t ready;
#define MORTAR_MMA4_BODY(GROUP)                                                                      \
    asm volatile(                                                                                    \
        "{\n.reg .pred q, p0, p1;\n.reg .b64 da, db;\n"                                              \
        "mbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n"                                    \
        "setp.eq.u32 p0, %12, 1;\n"                                                                  \
        "setp.eq.u32 p1, 1, 1;\n"                                                                    \
        "mov.b64 da, {%4, %11};\n mov.b64 db, {%8, %11};\n"                                          \
        "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%3], da, db, %13, p0;\n"                        \
        "mov.b64 da, {%5, %11};\n mov.b64 db, {%9, %11};\n"                                          \
        "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%3], da, db, %13, p1;\n"                        \
        "mov.b64 da, {%6, %11};\n mov.b64 db, {%10, %11};\n"                                         \
        "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%3], da, db, %13, p1;\n"                        \
        "mov.b64 da, {%7, %11};\n mov.b64 db, {%14, %11};\n"                                         \
        "tcgen05.mma.cta_group::" GROUP ".kind::f16 [%3], da, db, %13, p1;\n"                        \
        "selp.b32 %0, 1, 0, q;\n}\n"                                                                 \
        : "=r"(ready)                                                                                \
        : "r"(next_bar), "r"(next_parity), "r"(d_tmem), "r"(a_lo), "r"(a_lo + 2), "r"(a_lo + 4),    \
          "r"(a_lo + 6), "r"(b_lo), "r"(b_lo + 2), "r"(b_lo + 4), "r"(d_hi), "n"(FIRST_ACC ? 1 : 0), \
          "r"(idesc), "r"(b_lo + 6)                                                                  \
        : "memory")
    if (PAIR) MORTAR_MMA4_BODY("2");
    else MORTAR_MMA4_BODY("1");
#undef MORTAR_MMA4_BODY
    return ready != 0;
}
__device__ __forceinline__ void tc_mma_i8(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                          uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 da, db;\n"
        "setp.ne.b32 p, %6, 0;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate));
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(bar) : "memory");
}
// 32 accumulator columns of this thread's tensor-memory lane; tc_ld_wait() before the first use.
// The registers are in-out operands of the wait so that no use of them is scheduled above it.
__device__ __forceinline__ void tc_ld_wait(uint32_t (&r)[32]) {
    asm volatile("tcgen05.wait::ld.sync.aligned;\n"
        : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
          "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15]),
          "+r"(r[16]), "+r"(r[17]), "+r"(r[18]), "+r"(r[19]), "+r"(r[20]), "+r"(r[21]), "+r"(r[22]), "+r"(r[23]),
          "+r"(r[24]), "+r"(r[25]), "+r"(r[26]), "+r"(r[27]), "+r"(r[28]), "+r"(r[29]), "+r"(r[30]), "+r"(r[31])
        :: "memory");
}
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

__device__ __forceinline__ float rbf(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Two adjacent outputs of the epilogue with the reference's rounding points, in packed bf16:
// the reference's ops ARE bf16 ops (each rounds to nearest even), so after the fp32 scale and
// the fp32 silu the products are single bf16x2 multiplies.
template <bool SWIGLU, bool GATED>
__device__ __forceinline__ uint32_t finish2(float scale, float a0, float a1, float b0, float b1,
                                            bool live_a, bool live_b, float gate0, float gate1) {
    __nv_bfloat162 g2 = __floats2bfloat162_rn(live_a ? scale * a0 : 0.f, live_a ? scale * a1 : 0.f);
    if (!SWIGLU) return *reinterpret_cast<uint32_t *>(&g2);
    const __nv_bfloat162 u2 = __floats2bfloat162_rn(live_b ? scale * b0 : 0.f, live_b ? scale * b1 : 0.f);
    const float gx = __low2float(g2), gy = __high2float(g2);
    const __nv_bfloat162 s2 = __floats2bfloat162_rn(__fdividef(gx, 1.f + __expf(-gx)),
                                                    __fdividef(gy, 1.f + __expf(-gy)));
    __nv_bfloat162 h2 = __hmul2(s2, u2);
    if (GATED) {
        h2 = __hmul2(h2, __floats2bfloat162_rn(gate0, gate1));
        // a gate of zero (inactive group) yields an exact zero
        if (!(gate0 > 0.f)) h2.x = __float2bfloat16_rn(0.f);
        if (!(gate1 > 0.f)) h2.y = __float2bfloat16_rn(0.f);
    }
    return *reinterpret_cast<uint32_t *>(&h2);
}

// Flattened walk over the schedule steps of one pipe for every item of this CTA.
struct StepCursor {
    int item, s, s_end;
    __device__ __forceinline__ bool valid(const PrefillParams &p) const { return item < p.n_items; }
    __device__ __forceinline__ void enter(const PrefillParams &p, int n_super, int pipe) {
        // moves forward to the next item that has steps
        while (item < p.n_items) {
            const int panel = (item % n_super) * kPipes + pipe;
            s = __ldg(p.panel_step_ptr + panel);
            s_end = __ldg(p.panel_step_ptr + panel + 1);
            if (s < s_end) return;
            item += gridDim.x;
        }
    }
    __device__ __forceinline__ void start(const PrefillParams &p, int n_super, int pipe) {
        item = blockIdx.x; s = s_end = 0;
        enter(p, n_super, pipe);
    }
    __device__ __forceinline__ void next(const PrefillParams &p, int n_super, int pipe) {
        if (++s < s_end) return;
        item += gridDim.x;
        enter(p, n_super, pipe);
    }
};

// Drains one item's accumulators of one pipe: the epilogue of warp (pipe, quadrant q).
template <bool SWIGLU, bool GATED, bool I8>
__device__ __forceinline__ void epilogue_item(const PrefillParams &p, uint32_t taddr, int panel, long long row,
                                              bool in_range, uint32_t mask) {
    // int8 arm: the accumulators are int32 sums of (quantised activation x code); the row's
    // activation scale joins the per-matrix scale
    const float scale = I8 ? p.scale * (in_range ? __ldg(p.x_scale + row) : 0.f) : p.scale;
    constexpr int units = SWIGLU ? kPanelRows / 2 : kPanelRows;
    const bool tile_gates = GATED && (p.cluster_size % 16 == 0);     // one gate per 16-column tile
#pragma unroll 1
    for (int j = 0; j < units; j += 2) {                              // two output tile columns at a time
        uint32_t a[32], b[32];
        tc_ld32(taddr + j * 16, a);
        if (SWIGLU) tc_ld32(taddr + (units + j) * 16, b);
        tc_ld_wait(a);                                                  // both loads are in flight before the
        if (SWIGLU) tc_ld_wait(b);                                      // first wait; the second finds nothing pending
        const long long col0 = ((long long)panel * units + j) * 16;
        float tg[2] = {1.f, 1.f};
        if (GATED && tile_gates && in_range) {
            tg[0] = __ldg(p.gates + row * p.ld_gates + col0 / p.cluster_size);
            tg[1] = __ldg(p.gates + row * p.ld_gates + (col0 + 16) / p.cluster_size);
        }
        uint32_t packed[16];
#pragma unroll
        for (int e = 0; e < 32; e += 2) {
            const int jj = j + (e >> 4);
            const bool live_a = (mask >> jj) & 1u;
            const bool live_b = SWIGLU ? ((mask >> (units + jj)) & 1u) : true;
            float gate0 = tg[e >> 4], gate1 = tg[e >> 4];
            if (GATED && !tile_gates && in_range) {
                gate0 = __ldg(p.gates + row * p.ld_gates + (col0 + e) / p.cluster_size);
                gate1 = __ldg(p.gates + row * p.ld_gates + (col0 + e + 1) / p.cluster_size);
            }
            auto val = [](uint32_t bits) { return I8 ? __int2float_rn((int)bits) : __uint_as_float(bits); };
            packed[e >> 1] = finish2<SWIGLU, GATED>(scale, val(a[e]), val(a[e + 1]),
                                                    SWIGLU ? val(b[e]) : 0.f, SWIGLU ? val(b[e + 1]) : 0.f,
                                                    live_a, live_b, gate0, gate1);
        }
        if (in_range) {
            uint4 *dst = reinterpret_cast<uint4 *>(p.out + row * p.ld_out + col0);
            if (panel * units + j < p.total_units) {
                dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            }
            if (panel * units + j + 1 < p.total_units) {
                dst[2] = make_uint4(packed[8], packed[9], packed[10], packed[11]);
                dst[3] = make_uint4(packed[12], packed[13], packed[14], packed[15]);
            }
        }
    }
}

// I8 = false: bf16 activations x ternary codes expanded to bf16 (kind::f16, fp32 accumulators).
// I8 = true: int8 activations (quantised per row by quantize_rows_kernel) x codes expanded to
// int8 (kind::i8, int32 accumulators, K = 32 per MMA: a slot is a pair of tiles side by side).
template <bool I8>
__global__ void __launch_bounds__(kThreads, 1)
prefill_panel_kernel(const __grid_constant__ CUtensorMap tmap_x, const PrefillParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *sA = smem;                                          // kAStages x 16 KB, 1024-byte aligned
    uint8_t *sB = sA + kAStages * kAStage;                       // kPipes x kBStages x kBStage
    uint64_t *bars = reinterpret_cast<uint64_t *>(sB + kPipes * kBStages * kBStage);
    uint64_t *a_full = bars, *a_empty = a_full + kAStages;
    uint64_t *b_full = a_empty + kAStages;                       // [pipe][stage]
    uint64_t *b_empty = b_full + kPipes * kBStages;
    uint64_t *acc_full = b_empty + kPipes * kBStages, *acc_empty = acc_full + 1;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_super = p.n_panels / kPipes;                     // panel pairs

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kAStages; ++s) { mbar_init(smem_u32(&a_full[s]), 1); mbar_init(smem_u32(&a_empty[s]), kPipes); }
        for (int s = 0; s < kPipes * kBStages; ++s) { mbar_init(smem_u32(&b_full[s]), kDecodeThreads / 32); mbar_init(smem_u32(&b_empty[s]), 1); }
        mbar_init(smem_u32(acc_full), kPipes);
        mbar_init(smem_u32(acc_empty), kEpilogueThreads);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == kMmaWarp0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    volatile int *abort_flag = &abort_s;

    if (warp < kEpilogueWarps) {
        // ---------------- epilogue: warps 0..3 drain pipe 0, warps 4..7 pipe 1 ----------------
        const int q = warp & 3;                                       // tensor-memory lane quadrant
        const int pipe = warp >> 2;
        int it = 0;
        bool ok = true;
        const int units = p.swiglu ? kPanelRows / 2 : kPanelRows;
        (void)units;
        PF_DECL;
        for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++it) {
            const int panel = (item % n_super) * kPipes + pipe;
            const long long row = (long long)(item / n_super) * kRows + q * 32 + lane;
            const bool in_range = row < p.rows;
            const uint32_t mask = p.panel_mask[panel];
            PF_ACC(0);
            ok = mbar_wait_relaxed(smem_u32(acc_full), it & 1, abort_flag, 8);
            if (!ok) break;
            PF_ACC(1);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t taddr = tmem + pipe * kAccCols + ((uint32_t)(q * 32) << 16);
            if (!p.swiglu) epilogue_item<false, false, I8>(p, taddr, panel, row, in_range, mask);
            else if (p.gates == nullptr) epilogue_item<true, false, I8>(p, taddr, panel, row, in_range, mask);
            else epilogue_item<true, true, I8>(p, taddr, panel, row, in_range, mask);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            mbar_arrive(smem_u32(acc_empty));                         // accumulators drained
            PF_ACC(2);
        }
        PF_PUT(0, warp == 0 && lane == 0);
    } else if (warp == kMmaWarp0 || warp == kMmaWarp1) {
        // ---------------- MMA issue, one warp per pipe ----------------
        const int pipe = warp == kMmaWarp0 ? 0 : 1;
        uint64_t *bf = b_full + pipe * kBStages, *be = b_empty + pipe * kBStages;
        const uint8_t *bbase = sB + pipe * kBStages * kBStage;
        const uint32_t acc = tmem + pipe * kAccCols;
        // instruction descriptor of an N = 16 MMA: kind::f16, D fp32 (bit 4), A bf16 (bit 7), B bf16
        // (bit 10), both K-major, N>>3 at bit 17, M>>4 at bit 24; a run of len tiles adds (len-1)<<18
        // (kind::i8: D s32 = 2 at bit 4, A and B s8 = 1 at bits 7 and 10)
        constexpr uint32_t kIdesc16 = I8 ? ((2u << 4) | (1u << 7) | (1u << 10) | (2u << 17) | ((128u >> 4) << 24))
                                         : ((1u << 4) | (1u << 7) | (1u << 10) | (2u << 17) | ((128u >> 4) << 24));
        int g = 0, ga = -1, it = 0;
        bool ok = true;
        PF_DECL;
        for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++it) {
            const int panel = (item % n_super) * kPipes + pipe;
            const int n_steps = p.panel_step_ptr[panel + 1] - p.panel_step_ptr[panel];
            PF_ACC(0);
            ok = mbar_wait_relaxed(smem_u32(acc_empty), (it & 1) ^ 1u, abort_flag, 9);
            if (!ok) break;
            PF_ACC(1);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            for (int i = 0; i < n_steps; ++i, ++g) {
                const int bs = g % kBStages;
                // the decoders publish the step (tiles, run records, header) in the B stage
                ok = mbar_wait(smem_u32(&bf[bs]), (g / kBStages) & 1, abort_flag, 3);
                if (!ok) break;
                PF_ACC(2);
                const uint8_t *rec = bbase + bs * kBStage + kBTiles;
                const uint4 hdr = *reinterpret_cast<const uint4 *>(rec + kRunBytes);
                if (!(hdr.z & 0x40000000u)) {              // this step starts a new activation chunk
                    ++ga;
                    ok = mbar_wait(smem_u32(&a_full[ga % kAStages]), (ga / kAStages) & 1, abort_flag, 2);
                    if (!ok) break;
                }
                PF_ACC(3);
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                if (lane == 0) {
                    const int as = ga % kAStages;
                    const uint64_t a0 = make_smem_desc(smem_u32(sA + as * kAStage), 16, 1024, 2);
                    const uint64_t b0 = make_smem_desc(smem_u32(bbase + bs * kBStage), 128, 256, 0);
                    const uint32_t a_lo = (uint32_t)a0, a_hi = (uint32_t)(a0 >> 32);
                    const uint32_t b_lo = (uint32_t)b0, b_hi = (uint32_t)(b0 >> 32);
                    const uint4 *rr = reinterpret_cast<const uint4 *>(rec);
                    const int nrun = (int)hdr.y;
                    const uint32_t keep0 = hdr.w ? 0u : 1u;   // the panel's first MMA overwrites the accumulators
                    for (int r = 0; r < nrun; r += 8) {
                        const uint4 qv = rr[r >> 3];
                        const uint32_t ws[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            const uint32_t w = (k & 1) ? (ws[k >> 1] >> 16) : (ws[k >> 1] & 0xffffu);
                            if (r + k < nrun) {
                                if (I8) tc_mma_i8(acc + (w & 15u) * 16u, a_lo + ((w >> 10) & 3u) * 2u, a_hi,
                                                  b_lo + ((w >> 4) & 63u) * 32u, b_hi, kIdesc16 + ((w >> 12) << 18),
                                                  (r + k) ? 1u : keep0);
                                else tc_mma(acc + (w & 15u) * 16u, a_lo + ((w >> 10) & 3u) * 2u, a_hi,
                                            b_lo + ((w >> 4) & 63u) * 32u, b_hi, kIdesc16 + ((w >> 12) << 18),
                                            (r + k) ? 1u : keep0);
                            }
                        }
                    }
                    PF_ACC(4);
                    tc_commit(smem_u32(&be[bs]));          // B stage reusable once these MMAs retire
                    if (hdr.z & 0x80000000u) tc_commit(smem_u32(&a_empty[as]));   // last step on this chunk
                    PF_ACC(5);
                }
                __syncwarp();
            }
            if (!ok) break;
            if (lane == 0) {
                if (n_steps > 0) tc_commit(smem_u32(acc_full));
                else mbar_arrive(smem_u32(acc_full));
            }
            __syncwarp();
        }
        PF_PUT(8, pipe == 0 && lane == 0);
    } else if (warp == kTmaWarp) {
        // ---------------- TMA producer: the activation chunks pipe 0's steps name ----------------
        // (both panels of a pair list the same chunks)
        int ga = 0;
        bool ok = true;
        PF_DECL;
        StepCursor c;
        for (c.start(p, n_super, 0); c.valid(p) && ok; c.next(p, n_super, 0)) {
            const uint32_t meta = __ldg(p.step_meta + c.s);
            if (meta & 0x40000000u) continue;                        // reuses the chunk already requested
            const int row0 = (c.item / n_super) * kRows;
            const int as = ga % kAStages;
            PF_ACC(0);
            ok = mbar_wait_relaxed(smem_u32(&a_empty[as]), ((ga / kAStages) & 1) ^ 1u, abort_flag, 5);
            if (!ok) break;
            PF_ACC(1);
            if (lane == 0) {
                const uint32_t bar = smem_u32(&a_full[as]);
                mbar_arrive_expect_tx(bar, kAStage);
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                    "[%0], [%1, {%2, %3}], [%4];\n"
                    ::"r"(smem_u32(sA + as * kAStage)), "l"(&tmap_x),
                      "r"((int)(meta & 0x3fffu) * (I8 ? 128 : kChunkCols * 16)), "r"(row0), "r"(bar) : "memory");
            }
            __syncwarp();
            ++ga;
        }
        PF_ACC(0);
        PF_PUT(16, lane == 0);
    } else if (warp != kIdleWarp) {
        // ---------------- tile decode: warps 8, 9, 10, 12 pipe 0; 13, 14, 16, 17 pipe 1 ----------------
        const int di = warp - 8 - (warp > kMmaWarp0 ? 1 : 0) - (warp > kMmaWarp1 ? 1 : 0);
        const int pipe = di >> 2;
        const int td = (di & 3) * 32 + lane;
        uint64_t *bf = b_full + pipe * kBStages, *be = b_empty + pipe * kBStages;
        uint8_t *bbase = sB + pipe * kBStages * kBStage;
        int g = 0;
        bool ok = true;
        PF_DECL;
        // a step's record, fetched one step ahead of its expansion: meta word and offset two ahead
        auto fetch_info = [&](const StepCursor &c, uint32_t &meta, uint32_t &off) {
            meta = 0; off = 0;
            if (c.valid(p)) { meta = __ldg(p.step_meta + c.s); off = __ldg(p.step_off + c.s); }
        };
        // one row record = the codes of one tile row of a slot: a 32-bit word (bf16 arm: 16 codes)
        // or 16 bytes (int8 arm: 32 codes as nibbles)
        using Row = typename std::conditional<I8, uint4, uint32_t>::type;
        constexpr int kW = I8 ? kRowsPerThreadI8 : kWordsPerThread;
        auto fetch_words = [&](uint32_t meta, uint32_t off, Row (&w)[kW], uint4 &run) {
            const int ntile = (meta >> 14) & 63, nrun = (meta >> 20) & 63;
            const int run_units = (nrun + 7) >> 3;
            const uint8_t *rec = p.step_data + (size_t)off * 16;
            run = make_uint4(0, 0, 0, 0);
            if (td < run_units) run = __ldg(reinterpret_cast<const uint4 *>(rec + 16) + td);
            const Row *words = reinterpret_cast<const Row *>(rec + 16 + run_units * 16);
#pragma unroll
            for (int k = 0; k < kW; ++k) {
                const int idx = td + k * kDecodeThreads;
                if (idx < ntile * 16) w[k] = __ldg(words + idx);
            }
        };
        // Expands the step (cur, mc) held in (w, run) into its B stage; before that it requests the
        // following step's record (mn, on) into (wn, runn), so those loads are in flight while this
        // step waits for its stage and is expanded.  The two register sets swap roles from call to
        // call (no copy, so nothing waits for the loads before they are used).
        auto do_step = [&](uint32_t mc, const Row (&w)[kW], const uint4 &run,
                           bool have_next, uint32_t mn, uint32_t on, Row (&wn)[kW],
                           uint4 &runn) -> bool {
            const int bs = g % kBStages;
            if (have_next) fetch_words(mn, on, wn, runn);
            PF_ACC(0);
            if (!mbar_wait_relaxed(smem_u32(&be[bs]), ((g / kBStages) & 1) ^ 1u, abort_flag, 7)) return false;
            PF_ACC(3);
            uint8_t *bdst = bbase + bs * kBStage;
            const int ntile = (mc >> 14) & 63, nrun = (mc >> 20) & 63;
            if (td < ((nrun + 7) >> 3)) *reinterpret_cast<uint4 *>(bdst + kBTiles + td * 16) = run;
            if (td == kDecodeThreads - 1) {
                // header for the MMA warp: n_tiles, n_runs, meta, 1 if the step's first run is the
                // panel's initialising MMA (it overwrites the accumulators)
                *reinterpret_cast<uint4 *>(bdst + kBTiles + kRunBytes) = make_uint4(ntile, nrun, mc, (mc >> 29) & 1u);
            }
#pragma unroll
            for (int k = 0; k < kW; ++k) {
                const int idx = td + k * kDecodeThreads;
                if (idx < ntile * 16) {
                    const int tile = idx >> 4, row = idx & 15;
                    uint32_t o[8];
                    if constexpr (I8) {
                        // a nibble (stored value 0, 1, 2) selects the byte -1, 0, +1 of the table
                        const uint32_t ws[4] = {w[k].x, w[k].y, w[k].z, w[k].w};
#pragma unroll
                        for (int qq = 0; qq < 4; ++qq) {
                            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(o[2 * qq]) : "r"(0x000100ffu), "r"(0u), "r"(ws[qq]));
                            asm("prmt.b32 %0, %1, %2, %3;" : "=r"(o[2 * qq + 1]) : "r"(0x000100ffu), "r"(0u), "r"(ws[qq] >> 16));
                        }
                    } else {
#pragma unroll
                        for (int qq = 0; qq < 8; ++qq) o[qq] = mortar_decode_pair(w[k], qq);
                    }
                    uint8_t *d = bdst + tile * 512 + (row >> 3) * 256 + (row & 7) * 16;
                    *reinterpret_cast<uint4 *>(d) = make_uint4(o[0], o[1], o[2], o[3]);         // first 16 bytes of K
                    *reinterpret_cast<uint4 *>(d + 128) = make_uint4(o[4], o[5], o[6], o[7]);   // second 16 bytes of K
                }
            }
            // every lane orders its own stores before the tensor core's reads; one arrival per warp
            // (128 arrivals on one barrier word serialise)
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bf[bs]));
            PF_ACC(4);
            ++g;
            return true;
        };
        // cursors and (meta, offset) of the current step and the three after it
        StepCursor c[4];
        uint32_t m[4], o[4];
        c[0].start(p, n_super, pipe);
        fetch_info(c[0], m[0], o[0]);
        for (int k = 1; k < 4; ++k) {
            c[k] = c[k - 1];
            if (c[k].valid(p)) c[k].next(p, n_super, pipe);
            fetch_info(c[k], m[k], o[k]);
        }
        Row wa[kW], wb[kW];
        uint4 runa, runb;
        if (c[0].valid(p)) fetch_words(m[0], o[0], wa, runa);
        auto advance = [&]() {
#pragma unroll
            for (int k = 0; k < 3; ++k) { c[k] = c[k + 1]; m[k] = m[k + 1]; o[k] = o[k + 1]; }
            if (c[3].valid(p)) c[3].next(p, n_super, pipe);
            fetch_info(c[3], m[3], o[3]);
        };
        while (c[0].valid(p) && ok) {
            ok = do_step(m[0], wa, runa, c[1].valid(p), m[1], o[1], wb, runb);
            if (!ok) break;
            advance();
            if (!c[0].valid(p)) break;
            ok = do_step(m[0], wb, runb, c[1].valid(p), m[1], o[1], wa, runa);
            if (!ok) break;
            advance();
        }
        PF_PUT(24, pipe == 0 && td == 0);
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == kMmaWarp0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

std::mutex g_prefill_init_mutex;   // guards the first-use initialisation below
std::atomic<int> g_blocks_mode{0};  // block path: 0 = chosen per call, 1 = single CTAs, 2 = CTA pairs

int get_encode_fn(EncodeTiledFn *out) {
    static EncodeTiledFn cached = nullptr;
    std::lock_guard<std::mutex> lock(g_prefill_init_mutex);
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

// One launch of the panel kernel.  I8: x is int8 [rows][ldx] with per-row scales x_scale.
template <bool I8>
int linear_tc_impl(const mortar_sched *w, const void *x, int64_t ldx, int64_t rows, const float *x_scale,
                   void *out, int64_t ld_out, const float *gates, int64_t ld_gates,
                   int32_t cluster_size, void *stream) {
    if (!w || !x || !out || !w->panel_step_ptr || !w->panel_mask) return MORTAR_ERR_NULL;
    if (I8 && !x_scale) return MORTAR_ERR_NULL;
    if (w->n_steps > 0 && (!w->step_data || !w->step_off || !w->step_meta)) return MORTAR_ERR_NULL;
    if (w->tile_rows <= 0 || w->tile_cols <= 0 || w->n_panels <= 0 || rows < 0) return MORTAR_ERR_SHAPE;
    if (w->arith != (I8 ? 1 : 0)) return MORTAR_ERR_DTYPE;       // schedule built for the other arm
    const int K = w->tile_cols * 16;
    const int units = w->swiglu ? w->tile_rows / 2 : w->tile_rows;
    if (ldx < K || ld_out < (int64_t)units * 16) return MORTAR_ERR_SHAPE;
    const int x_elems16 = I8 ? 16 : 8;                          // elements per 16 bytes of x
    if (!aligned_to(x, 16) || (ldx % x_elems16) || !aligned_to(out, 16) || (ld_out % 8)) return MORTAR_ERR_ALIGN;
    if (!aligned_to(w->step_data, 16)) return MORTAR_ERR_ALIGN;
    if (gates && (cluster_size <= 0 || !w->swiglu)) return MORTAR_ERR_SHAPE;
    if (rows == 0) return MORTAR_OK;
    const int64_t row_blocks = (rows + kRows - 1) / kRows;
    if (w->n_panels % kPipes) return MORTAR_ERR_SHAPE;          // the builder pads to pairs
    const int64_t n_items = row_blocks * (w->n_panels / kPipes);
    if (n_items > 0x7fffffffLL || rows > 0x7fffffffLL) return MORTAR_ERR_CAPACITY;

    EncodeTiledFn encode;
    int rc = get_encode_fn(&encode);
    if (rc != MORTAR_OK) return rc;
    alignas(64) CUtensorMap tmap;
    const cuuint64_t gdim[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)ldx * (I8 ? 1 : 2)};
    const cuuint32_t box[2] = {I8 ? 128u : 64u, (cuuint32_t)kRows};    // 128 bytes wide either way
    const cuuint32_t estride[2] = {1, 1};
    CUresult cr = encode(&tmap, I8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                         const_cast<void *>(x), gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                         CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        mortar_set_cuda_error("cuTensorMapEncodeTiled", "failed to encode the activation tensor map");
        return MORTAR_ERR_CUDA;
    }

    int dev = 0;
    MORTAR_CUDA_CHECK(cudaGetDevice(&dev));
    static int sm_count[64] = {0};                               // one table per arm
    if (dev < 0 || dev >= 64) return MORTAR_ERR_CAPACITY;
    int sms = 0;
    {
        std::lock_guard<std::mutex> lock(g_prefill_init_mutex);
        if (sm_count[dev] == 0) {
            int v = 0;
            MORTAR_CUDA_CHECK(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(prefill_panel_kernel<I8>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
            sm_count[dev] = v;
        }
        sms = sm_count[dev];
    }
    PrefillParams p;
    p.step_data = reinterpret_cast<const uint8_t *>(w->step_data);
    p.step_off = w->step_off;
    p.step_meta = w->step_meta;
    p.panel_step_ptr = w->panel_step_ptr;
    p.panel_mask = w->panel_mask;
    p.n_panels = w->n_panels;
    p.n_items = (int)n_items;
    p.swiglu = w->swiglu;
    p.total_units = units;
    p.rows = rows;
    p.out = reinterpret_cast<__nv_bfloat16 *>(out);
    p.ld_out = ld_out;
    p.scale = __bfloat162float(__float2bfloat16_rn(w->scale));
    p.x_scale = x_scale;
    p.gates = gates;
    p.ld_gates = ld_gates;
    p.cluster_size = cluster_size > 0 ? cluster_size : 1;
    const unsigned grid = (unsigned)(n_items < sms ? n_items : sms);
    prefill_panel_kernel<I8><<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(tmap, p);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

// ---------------------------------------------------------------------------------------------
// Block path: topologies made of (mostly) full 128 x 128 blocks -- the granularity the reference
// carves at (carve(blocking=128), block_sparse.py:810-907).  The kept blocks are held expanded
// (codes as bf16, one [128 outputs][128 inputs] block after the other, what the reference keeps as
// `mortar_data`), so a block is a plain tensor-core operand that TMA brings in: no decode stage,
// N = 256 MMAs, and 256 accumulator columns per item leave room for two accumulator sets, so the
// epilogue of an item runs under the MMAs of the next one.
//
// Item = 128 activation rows x a PAIR of block rows (SwiGLU: gate block row g and the up block row
// of the same hidden columns; linear: block rows 2p, 2p+1); the pair's step list names, per block
// column either of them keeps, the block index of each (or -1).  Per step and half (K = 64): the
// TMA warp loads the activation chunk [128 x 64] and the present blocks' [128 x 64] halves; the
// MMA warp issues one N = 256 MMA per 16 features when both blocks are present (they lie back to
// back in the stage), else N = 128 into the present half.  Eight epilogue warps (two per
// tensor-memory lane quadrant, each half of the columns) finish as the tile path does.
constexpr int kBkStages = 4;
constexpr int kBkA = kRows * 128;                    // [128 rows][64 features] bf16
constexpr int kBkB = 128 * 128;                      // [128 outputs][64 features] of one block
constexpr int kBkStage = kBkA + 2 * kBkB;            // 48 KB
constexpr int kBkEpiWarps = 8;
constexpr int kBkThreads = 32 * (2 + kBkEpiWarps);   // TMA warp, MMA warp, epilogue warps
constexpr int kBkMaxSteps = 1024, kBkMaxPairs = 511;   // step lists up to this size are staged in shared memory
constexpr int kBkSmemBytes = kBkStages * kBkStage + (2 * kBkStages + 4) * 8 + kBkMaxSteps * 16 + (kBkMaxPairs + 1) * 4 +
                             1024 /*align*/;
static_assert(kBkSmemBytes <= 227 * 1024, "shared memory budget");

struct BlockParams {
    const int *pair_ptr;          // [n_pairs + 1] first step of every pair of block rows
    const int4 *steps;            // [n_steps] {block column, block index of the first row or -1, of the second or -1, 0}
    int n_pairs;
    int n_steps;
    int n_items;                  // n_pairs * row blocks
    int swiglu;
    int n_out;                    // output columns: hidden width (SwiGLU) or out_features (linear)
    long long rows;
    __nv_bfloat16 *out;
    long long ld_out;
    float scale;
    const float *gates;
    long long ld_gates;
    int cluster_size;
};

// Finishes columns [c0, c0 + 32) of one accumulator set for this thread's row.
template <bool SWIGLU, bool GATED>
__device__ __forceinline__ void block_epilogue_chunk(const BlockParams &p, uint32_t taddr, long long row, bool in_range,
                                                     long long col0, int c0, bool live_a, bool live_b) {
    // an accumulator half that received no block holds undefined values: zeros stand in for it, so the
    // arithmetic below needs no per-element select
    uint32_t a[32], b[32];
    if (live_a) {
        tc_ld32(taddr + c0, a);
    } else {
#pragma unroll
        for (int e = 0; e < 32; ++e) a[e] = 0u;
    }
    if (SWIGLU) {
        if (live_b) {
            tc_ld32(taddr + 128 + c0, b);
        } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) b[e] = 0u;
        }
    }
    tc_ld_wait(a);
    if (SWIGLU) tc_ld_wait(b);
    const bool tile_gates = GATED && (p.cluster_size % 16 == 0);
    float tg[2] = {1.f, 1.f};
    if (GATED && tile_gates && in_range) {       // columns past the hidden width (a padded last pair) have no gate
        if (col0 < p.n_out) tg[0] = __ldg(p.gates + row * p.ld_gates + col0 / p.cluster_size);
        if (col0 + 16 < p.n_out) tg[1] = __ldg(p.gates + row * p.ld_gates + (col0 + 16) / p.cluster_size);
    }
    uint32_t packed[16];
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
        float gate0 = tg[e >> 4], gate1 = tg[e >> 4];
        if (GATED && !tile_gates && in_range && col0 + e + 1 < p.n_out) {
            gate0 = __ldg(p.gates + row * p.ld_gates + (col0 + e) / p.cluster_size);
            gate1 = __ldg(p.gates + row * p.ld_gates + (col0 + e + 1) / p.cluster_size);
        }
        packed[e >> 1] = finish2<SWIGLU, GATED>(p.scale, __uint_as_float(a[e]), __uint_as_float(a[e + 1]),
                                                SWIGLU ? __uint_as_float(b[e]) : 0.f, SWIGLU ? __uint_as_float(b[e + 1]) : 0.f,
                                                true, true, gate0, gate1);
    }
    if (in_range) {
        uint4 *dst = reinterpret_cast<uint4 *>(p.out + row * p.ld_out + col0);
        if (col0 < p.n_out) {
            dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
        if (col0 + 16 < p.n_out) {
            dst[2] = make_uint4(packed[8], packed[9], packed[10], packed[11]);
            dst[3] = make_uint4(packed[12], packed[13], packed[14], packed[15]);
        }
    }
}

__global__ void __launch_bounds__(kBkThreads, 1)
prefill_blocks_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                      const BlockParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *stages = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *full = reinterpret_cast<uint64_t *>(stages + kBkStages * kBkStage), *empty = full + kBkStages;
    uint64_t *acc_full = empty + kBkStages, *acc_empty = acc_full + 2;
    int4 *steps_s = reinterpret_cast<int4 *>(acc_empty + 2);
    int *pairs_s = reinterpret_cast<int *>(steps_s + kBkMaxSteps);
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    // the step lists are read by three roles for every item: keep them in shared memory when they fit
    const bool cached = p.n_steps <= kBkMaxSteps && p.n_pairs <= kBkMaxPairs;
    if (cached) {
        for (int i = threadIdx.x; i < p.n_steps; i += kBkThreads) steps_s[i] = __ldg(p.steps + i);
        for (int i = threadIdx.x; i <= p.n_pairs; i += kBkThreads) pairs_s[i] = __ldg(p.pair_ptr + i);
    }
    const int4 *steps = cached ? steps_s : p.steps;
    const int *pair_ptr = cached ? pairs_s : p.pair_ptr;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kBkStages; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&acc_full[s]), 1); mbar_init(smem_u32(&acc_empty[s]), kBkEpiWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
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
        // ---------------- TMA producer: one thread ----------------
        // Same shape as the MMA role: per-step values hoisted, the poll of the next stage's `empty`
        // barrier issued before the loads of the current one.
        if (lane == 0) {
            const uint32_t full0 = smem_u32(&full[0]), empty0 = smem_u32(&empty[0]), stage0 = smem_u32(stages);
            int g = 0;
            bool ok = true;
            bool ready = mbar_try_wait(empty0, 1u);
            for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x) {
                const int pair = item % p.n_pairs, row0 = (item / p.n_pairs) * kRows;
                const int s_beg = pair_ptr[pair], s_end = pair_ptr[pair + 1];
                int4 s_next = steps[s_beg < s_end ? s_beg : 0];
                for (int st = s_beg; st < s_end && ok; ++st, g += 2) {
                    const int4 s = s_next;
                    s_next = steps[st + 1 < s_end ? st + 1 : st];
                    const uint32_t bytes = kBkA + (s.y >= 0 ? kBkB : 0) + (s.z >= 0 ? kBkB : 0);
                    const uint32_t odd = ((uint32_t)g >> 1) & 1u, parity = (((uint32_t)g >> 2) & 1u) ^ 1u;
                    const int xcol = s.x * 128, yrow = s.y * 128, zrow = s.z * 128;
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t sg = odd * 2u + (uint32_t)h;
                        if (!ready) ok = mbar_wait_relaxed(empty0 + sg * 8u, parity, abort_flag, 5);
                        if (!ok) break;
                        // next stage: the pair's second stage, or the first stage of the other pair (whose phase
                        // flips when this pair is the second one)
                        ready = h == 0 ? mbar_try_wait(empty0 + (sg + 1u) * 8u, parity)
                                       : mbar_try_wait(empty0 + (odd ^ 1u) * 16u, parity ^ odd);
                        const uint32_t bar = full0 + sg * 8u;
                        const uint32_t dst = stage0 + sg * (uint32_t)kBkStage;
                        mbar_arrive_expect_tx(bar, bytes);
                        asm volatile(
                            "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                            "[%0], [%1, {%2, %3}], [%4];\n"
                            ::"r"(dst), "l"(&tmap_x), "r"(xcol + h * 64), "r"(row0), "r"(bar) : "memory");
                        if (s.y >= 0)
                            asm volatile(
                                "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                                "[%0], [%1, {%2, %3}], [%4];\n"
                                ::"r"(dst + kBkA), "l"(&tmap_w), "r"(h * 64), "r"(yrow), "r"(bar) : "memory");
                        if (s.z >= 0)
                            asm volatile(
                                "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
                                "[%0], [%1, {%2, %3}], [%4];\n"
                                ::"r"(dst + kBkA + kBkB), "l"(&tmap_w), "r"(h * 64), "r"(zrow), "r"(bar) : "memory");
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue: one thread ----------------
        // The issuing thread's own instruction stream is the critical path (the MMA queue holds only
        // two or three instructions, so every cycle the thread spends between MMAs beyond that is a
        // cycle the tensor pipe idles): everything a step decides is decided once per step, the
        // four MMAs of a stage are straight-line code, and the other lanes stay out of the loop.
        // kind::f16, D fp32, A and B bf16, both K-major; N >> 3 at bit 17, M >> 4 at bit 24
        constexpr uint32_t kIdescBase = (1u << 4) | (1u << 7) | (1u << 10) | ((128u >> 4) << 24);
        constexpr uint32_t kIdesc128 = kIdescBase | ((128u >> 3) << 17), kIdesc256 = kIdescBase | ((256u >> 3) << 17);
        if (lane == 0) {
            const uint64_t d0 = make_smem_desc(smem_u32(stages), 16, 1024, 2);
            const uint32_t a_lo0 = (uint32_t)d0, d_hi = (uint32_t)(d0 >> 32);   // stage 0; only the address field changes
            const uint32_t full0 = smem_u32(&full[0]), empty0 = smem_u32(&empty[0]);
            int g = 0, it = 0;
            bool ok = true;
            // The poll of a stage's barrier is issued one stage ahead, so its latency runs under the
            // MMAs of the stage before; a first poll that fails falls back to the bounded wait.
            bool ready = mbar_try_wait(full0, 0u);
            for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++it) {
                const int pair = item % p.n_pairs, buf = it & 1;
                if (!mbar_try_wait(smem_u32(&acc_empty[buf]), ((it >> 1) & 1) ^ 1u))
                    ok = mbar_wait_relaxed(smem_u32(&acc_empty[buf]), ((it >> 1) & 1) ^ 1u, abort_flag, 9);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t acc = tmem + buf * kAccCols;
                bool have_a = false, have_b = false;           // the halves hold defined values
                const int s_beg = pair_ptr[pair], s_end = pair_ptr[pair + 1];
                int4 s_next = steps[s_beg < s_end ? s_beg : 0];
                for (int st = s_beg; st < s_end && ok; ++st, g += 2) {
                    const int4 s = s_next;
                    s_next = steps[st + 1 < s_end ? st + 1 : st];          // the next step's record, ahead of its use
                    const bool ya = s.y >= 0, zb = s.z >= 0;
                    const bool wide = ya && zb && have_a == have_b;       // one N = 256 MMA covers both blocks
                    const bool two = ya && zb && !wide;                    // different accumulate states: two N = 128 MMAs
                    const uint32_t d1 = acc + (ya ? 0u : 128u);
                    const uint32_t idesc1 = wide ? kIdesc256 : kIdesc128;
                    const bool fresh = !(ya ? have_a : have_b);
                    // a step takes two consecutive stages, the first of them stage 0 or 2
                    const uint32_t odd = ((uint32_t)g >> 1) & 1u, parity = ((uint32_t)g >> 2) & 1u;
                    const uint32_t bar_f = full0 + odd * 16u, bar_e = empty0 + odd * 16u;
                    const uint32_t a_lo = a_lo0 + odd * (uint32_t)(2 * kBkStage >> 4);
                    const uint32_t b_lo = a_lo + (kBkA >> 4) + (ya ? 0u : (uint32_t)(kBkB >> 4));
                    constexpr uint32_t kS = kBkStage >> 4;
                    // first half
                    if (!ready) ok = mbar_wait(bar_f, parity, abort_flag, 2);
                    if (!ok) break;
                    if (!two) {
                        ready = fresh ? tc_poll_mma4<false, false>(bar_f + 8u, parity, d1, a_lo, b_lo, d_hi, idesc1)
                                      : tc_poll_mma4<true, false>(bar_f + 8u, parity, d1, a_lo, b_lo, d_hi, idesc1);
                    } else {
                        ready = mbar_try_wait(bar_f + 8u, parity);
                        uint32_t f1 = have_a ? 1u : 0u, f2 = have_b ? 1u : 0u;
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            tc_mma(acc, a_lo + kk * 2, d_hi, b_lo + kk * 2, d_hi, kIdesc128, f1);
                            tc_mma(acc + 128, a_lo + kk * 2, d_hi, b_lo + (uint32_t)(kBkB >> 4) + kk * 2, d_hi, kIdesc128, f2);
                            f1 = f2 = 1u;
                        }
                    }
                    tc_commit(bar_e);
                    // second half: the next stage; the poll after it goes to the stage the next step starts with
                    if (!ready) ok = mbar_wait(bar_f + 8u, parity, abort_flag, 2);
                    if (!ok) break;
                    if (!two) {
                        ready = tc_poll_mma4<true, false>(full0 + (odd ^ 1u) * 16u, parity ^ odd, d1, a_lo + kS, b_lo + kS, d_hi, idesc1);
                    } else {
                        ready = mbar_try_wait(full0 + (odd ^ 1u) * 16u, parity ^ odd);
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk) {
                            tc_mma_lit<true>(acc, a_lo + kS + kk * 2, d_hi, b_lo + kS + kk * 2, d_hi, kIdesc128);
                            tc_mma_lit<true>(acc + 128, a_lo + kS + kk * 2, d_hi, b_lo + kS + (uint32_t)(kBkB >> 4) + kk * 2, d_hi, kIdesc128);
                        }
                    }
                    tc_commit(bar_e + 8u);
                    have_a |= ya;
                    have_b |= zb;
                }
                if (!ok) break;
                if (s_end > s_beg) tc_commit(smem_u32(&acc_full[buf]));
                else mbar_arrive(smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // ---------------- epilogue: warps 2..9; lane quadrant = warp % 4, column half = (warp - 2) / 4 ----------------
        const int q = warp & 3, ch = (warp - 2) >> 2;
        int it = 0;
        bool ok = true;
        for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++it) {
            const int pair = item % p.n_pairs, buf = it & 1;
            const long long row = (long long)(item / p.n_pairs) * kRows + q * 32 + lane;
            const bool in_range = row < p.rows;
            // which of the two block rows received a block at all
            bool live_a = false, live_b = false;
            const int s_end = pair_ptr[pair + 1];
            for (int st = pair_ptr[pair]; st < s_end; ++st) {
                const int4 s = steps[st];
                live_a |= s.y >= 0;
                live_b |= s.z >= 0;
            }
            ok = mbar_wait_relaxed(smem_u32(&acc_full[buf]), (it >> 1) & 1, abort_flag, 8);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t taddr = tmem + buf * kAccCols + ((uint32_t)(q * 32) << 16);
            if (p.swiglu) {
                // hidden columns [128 pair, +128): gate sums in accumulator columns 0..127, up sums in 128..255
#pragma unroll 1
                for (int c0 = ch * 64; c0 < ch * 64 + 64; c0 += 32) {
                    const long long col0 = (long long)pair * 128 + c0;
                    if (p.gates == nullptr) block_epilogue_chunk<true, false>(p, taddr, row, in_range, col0, c0, live_a, live_b);
                    else block_epilogue_chunk<true, true>(p, taddr, row, in_range, col0, c0, live_a, live_b);
                }
            } else {
#pragma unroll 1
                for (int c0 = ch * 128; c0 < ch * 128 + 128; c0 += 32) {
                    const long long col0 = (long long)pair * 256 + c0;
                    block_epilogue_chunk<false, false>(p, taddr, row, in_range, col0, c0, c0 < 128 ? live_a : live_b, true);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

// ---------------------------------------------------------------------------------------------
// Block path on CTA pairs (tcgen05 cta_group::2).  A cluster of two CTAs works on 256 activation
// rows (128 each) against one pair of block rows: the MMA has M = 256 and its B operand is split
// between the two CTAs' shared memories, so each CTA stages and reads only half of every block
// (a quarter less traffic from L2 and through shared memory per FLOP) and one instruction drives
// both SMs' tensor cores (half the MMA instructions per FLOP for the one issuing thread).  The
// smaller stages leave room for six, three steps in flight, which lets a step hang on ONE pair of
// barriers.  Measured against the single-CTA kernel: 8% faster on a dense topology, 7% on ragged
// 128-blocks.
//
// Per step (one block column of the pair) and half (K = 64) each CTA loads its own [128 x 64]
// activation chunk and its share of the B operand:
//   both blocks present and in the same accumulate state: one N = 256 MMA per 16 features whose
//     B rows 0..127 are the first block (held by CTA 0) and 128..255 the second (held by CTA 1);
//   otherwise one N = 128 MMA per present block, whose B rows 0..63 are held by CTA 0 and 64..127
//     by CTA 1: every CTA loads 64 rows of each present block (first block at offset 0, second at
//     8 KB of the B region).
// All loads of a step complete on CTA 0's `full` barrier of the stage pair (its producer posts the
// byte count of both CTAs and both halves); one thread of CTA 0 issues for the pair and commits to
// the `empty` and accumulator barriers of both CTAs; the epilogue warps of both CTAs release an accumulator set on CTA 0's
// barrier.  Every wait is bounded as in the single-CTA kernel.
constexpr int kB2Stages = 6;
constexpr int kB2B = 128 * 128;                      // this CTA's share of the step's B operand
constexpr int kB2Stage = kBkA + kB2B;                // 32 KB
constexpr int kB2SmemBytes = kB2Stages * kB2Stage + (2 * kB2Stages + 4) * 8 + kBkMaxSteps * 16 + (kBkMaxPairs + 1) * 4 +
                             1024 /*align*/;
static_assert(kB2SmemBytes <= 227 * 1024, "shared memory budget");

__device__ __forceinline__ uint32_t cluster_cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(r));
    return r;
}
// shared::cluster address of the same shared-memory offset in CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_bar) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];\n" ::"r"(cluster_bar) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;\n" ::: "memory");
}
__device__ __forceinline__ void tc_mma_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                            uint32_t b_hi, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 da, db;\n"
        "setp.ne.b32 p, %6, 0;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate));
}
template <bool ACC>
__device__ __forceinline__ void tc_mma_pair_lit(uint32_t d_tmem, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo,
                                                uint32_t b_hi, uint32_t idesc) {
    asm volatile(
        "{\n.reg .pred p;\n.reg .b64 da, db;\n"
        "setp.eq.u32 p, %6, 1;\n"
        "mov.b64 da, {%1, %2};\n"
        "mov.b64 db, {%3, %4};\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %5, p;\n}\n"
        ::"r"(d_tmem), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "n"(ACC ? 1 : 0));
}
__device__ __forceinline__ void tc_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(cluster_bar) : "memory");
}
// TMA tile load into this CTA's shared memory that completes on a barrier of either CTA of the pair
__device__ __forceinline__ void tma_load_pair(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t cluster_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%2, %3}], [%4];\n"
        ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(cluster_bar) : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kBkThreads, 1)
prefill_blocks_pair_kernel(const __grid_constant__ CUtensorMap tmap_x, const __grid_constant__ CUtensorMap tmap_w,
                           const __grid_constant__ CUtensorMap tmap_wh, const BlockParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *stages = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *full = reinterpret_cast<uint64_t *>(stages + kB2Stages * kB2Stage), *empty = full + kB2Stages;
    uint64_t *acc_full = empty + kB2Stages, *acc_empty = acc_full + 2;
    int4 *steps_s = reinterpret_cast<int4 *>(acc_empty + 2);
    int *pairs_s = reinterpret_cast<int *>(steps_s + kBkMaxSteps);
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_cta_rank();
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;

    const bool cached = p.n_steps <= kBkMaxSteps && p.n_pairs <= kBkMaxPairs;
    if (cached) {
        for (int i = threadIdx.x; i < p.n_steps; i += kBkThreads) steps_s[i] = __ldg(p.steps + i);
        for (int i = threadIdx.x; i <= p.n_pairs; i += kBkThreads) pairs_s[i] = __ldg(p.pair_ptr + i);
    }
    const int4 *steps = cached ? steps_s : p.steps;
    const int *pair_ptr = cached ? pairs_s : p.pair_ptr;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kB2Stages; ++s) { mbar_init(smem_u32(&full[s]), 1); mbar_init(smem_u32(&empty[s]), 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(smem_u32(&acc_full[s]), 1); mbar_init(smem_u32(&acc_empty[s]), 2 * kBkEpiWarps); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        // the same warp of both CTAs allocates (and later frees) the pair's tensor memory
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_s)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();                                        // barriers of both CTAs are initialised
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = tmem_base_s;
    volatile int *abort_flag = &abort_s;

    if (warp == 0) {
        // ---------------- TMA producer: one thread in each CTA ----------------
        if (lane == 0) {
            const uint32_t full0 = smem_u32(&full[0]), full0_lead = map_to_cta(full0, 0);
            const uint32_t empty0 = smem_u32(&empty[0]), stage0 = smem_u32(stages);
            uint32_t sp = 0u, parity = 1u;                     // stage pair and the phase its `empty` barriers are waited in
            bool ok = true;
            bool ready = mbar_try_wait(empty0, 1u);
            for (int item = cluster_id; item < p.n_items && ok; item += n_clusters) {
                const int pair = item % p.n_pairs, row0 = (item / p.n_pairs) * (2 * kRows) + (int)rank * kRows;
                bool have_a = false, have_b = false;
                const int s_beg = pair_ptr[pair], s_end = pair_ptr[pair + 1];
                int4 s_next = steps[s_beg < s_end ? s_beg : 0];
                for (int st = s_beg; st < s_end && ok; ++st) {
                    const int4 s = s_next;
                    s_next = steps[st + 1 < s_end ? st + 1 : st];
                    const bool ya = s.y >= 0, zb = s.z >= 0;
                    const bool wide = ya && zb && have_a == have_b;
                    const uint32_t b_bytes = wide ? (uint32_t)kB2B : (uint32_t)(ya + zb) * (kB2B / 2);
                    const int xcol = s.x * 128;
                    const int yrow = wide ? (rank == 0 ? s.y : s.z) * 128 : s.y * 128 + (int)rank * 64;
                    const int zrow = s.z * 128 + (int)rank * 64;
                    const uint32_t sp_next = sp == 2u ? 0u : sp + 1u, parity_next = sp == 2u ? parity ^ 1u : parity;
                    // both stages of the step hang on the stage pair's first barriers
                    if (!ready) ok = mbar_wait_relaxed(empty0 + sp * 16u, parity, abort_flag, 5);
                    if (!ok) break;
                    ready = mbar_try_wait(empty0 + sp_next * 16u, parity_next);
                    const uint32_t bar = full0_lead + sp * 16u;
                    if (rank == 0) mbar_arrive_expect_tx(full0 + sp * 16u, 4u * (kBkA + b_bytes));
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t sg = sp * 2u + (uint32_t)h;
                        const uint32_t dst = stage0 + sg * (uint32_t)kB2Stage;
                        tma_load_pair(dst, &tmap_x, xcol + h * 64, row0, bar);
                        if (wide) {
                            tma_load_pair(dst + kBkA, &tmap_w, h * 64, yrow, bar);
                        } else {
                            if (ya) tma_load_pair(dst + kBkA, &tmap_wh, h * 64, yrow, bar);
                            if (zb) tma_load_pair(dst + kBkA + kB2B / 2, &tmap_wh, h * 64, zrow, bar);
                        }
                    }
                    sp = sp_next;
                    parity = parity_next;
                    have_a |= ya;
                    have_b |= zb;
                }
            }
        }
    } else if (warp == 1) {
        if (rank == 0 && lane == 0) {
            // ---------------- MMA issue: one thread of CTA 0 for the pair ----------------
            // kind::f16, D fp32, A and B bf16, both K-major; N >> 3 at bit 17, M >> 4 at bit 24 (M = 256 over the pair)
            constexpr uint32_t kIdescBase = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 4) << 24);
            constexpr uint32_t kIdesc128 = kIdescBase | ((128u >> 3) << 17), kIdesc256 = kIdescBase | ((256u >> 3) << 17);
            const uint64_t d0 = make_smem_desc(smem_u32(stages), 16, 1024, 2);
            const uint32_t a_lo0 = (uint32_t)d0, d_hi = (uint32_t)(d0 >> 32);
            const uint32_t full0 = smem_u32(&full[0]), empty0 = smem_u32(&empty[0]);
            const uint32_t empty0_peer = map_to_cta(empty0, 1);
            int it = 0;
            uint32_t sp = 0u, parity = 0u;                     // stage pair (stages 2sp, 2sp+1) and its phase
            bool ok = true;
            bool ready = mbar_try_wait(full0, 0u);             // polls run one stage ahead, as in the single-CTA kernel
            for (int item = cluster_id; item < p.n_items && ok; item += n_clusters, ++it) {
                const int pair = item % p.n_pairs, buf = it & 1;
                if (!mbar_try_wait(smem_u32(&acc_empty[buf]), ((it >> 1) & 1) ^ 1u))
                    ok = mbar_wait_relaxed(smem_u32(&acc_empty[buf]), ((it >> 1) & 1) ^ 1u, abort_flag, 9);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t acc = tmem + buf * kAccCols;
                bool have_a = false, have_b = false;
                const int s_beg = pair_ptr[pair], s_end = pair_ptr[pair + 1];
                int4 s_next = steps[s_beg < s_end ? s_beg : 0];
                for (int st = s_beg; st < s_end && ok; ++st) {
                    const int4 s = s_next;
                    s_next = steps[st + 1 < s_end ? st + 1 : st];
                    const bool ya = s.y >= 0, zb = s.z >= 0;
                    const bool wide = ya && zb && have_a == have_b;
                    const bool two = ya && zb && !wide;
                    // N = 128: the first block's share lies at the start of the B region, the second's 8 KB in
                    const uint32_t d1 = acc + (ya ? 0u : 128u);
                    const uint32_t idesc1 = wide ? kIdesc256 : kIdesc128;
                    const bool fresh = !(ya ? have_a : have_b);
                    const uint32_t bar_f = full0 + sp * 16u, bar_e = empty0 + sp * 16u, bar_ep = empty0_peer + sp * 16u;
                    const uint32_t a_lo = a_lo0 + sp * (uint32_t)(2 * kB2Stage >> 4);
                    const uint32_t b_lo = a_lo + (uint32_t)(kBkA >> 4) + (ya ? 0u : (uint32_t)(kB2B >> 5));
                    constexpr uint32_t kS = kB2Stage >> 4, kZ = kB2B >> 5;
                    const uint32_t sp_next = sp == 2u ? 0u : sp + 1u, parity_next = sp == 2u ? parity ^ 1u : parity;
                    // both stages of the step hang on the stage pair's first barriers: one wait, eight MMAs, one
                    // commit per CTA (with three stage pairs in flight this measured 4-6% faster than a barrier per
                    // stage; with the two pairs of the single-CTA kernel it measured slower); the poll goes to the
                    // stage pair the next step takes
                    if (!ready) ok = mbar_wait(bar_f, parity, abort_flag, 2);
                    if (!ok) break;
                    if (!two) {
                        ready = fresh ? tc_poll_mma4<false, true>(full0 + sp_next * 16u, parity_next, d1, a_lo, b_lo, d_hi, idesc1)
                                      : tc_poll_mma4<true, true>(full0 + sp_next * 16u, parity_next, d1, a_lo, b_lo, d_hi, idesc1);
                        tc_mma_pair_lit<true>(d1, a_lo + kS, d_hi, b_lo + kS, d_hi, idesc1);
                        tc_mma_pair_lit<true>(d1, a_lo + kS + 2, d_hi, b_lo + kS + 2, d_hi, idesc1);
                        tc_mma_pair_lit<true>(d1, a_lo + kS + 4, d_hi, b_lo + kS + 4, d_hi, idesc1);
                        tc_mma_pair_lit<true>(d1, a_lo + kS + 6, d_hi, b_lo + kS + 6, d_hi, idesc1);
                    } else {
                        ready = mbar_try_wait(full0 + sp_next * 16u, parity_next);
                        uint32_t f1 = have_a ? 1u : 0u, f2 = have_b ? 1u : 0u;
#pragma unroll
                        for (int kk = 0; kk < 8; ++kk) {
                            const uint32_t o = (uint32_t)(kk >> 2) * kS + (uint32_t)(kk & 3) * 2u;
                            tc_mma_pair(acc, a_lo + o, d_hi, b_lo + o, d_hi, kIdesc128, f1);
                            tc_mma_pair(acc + 128, a_lo + o, d_hi, b_lo + kZ + o, d_hi, kIdesc128, f2);
                            f1 = f2 = 1u;
                        }
                    }
                    tc_commit_pair(bar_e);
                    tc_commit_pair(bar_ep);
                    sp = sp_next;
                    parity = parity_next;
                    have_a |= ya;
                    have_b |= zb;
                }
                if (!ok) break;
                if (s_end > s_beg) {
                    tc_commit_pair(smem_u32(&acc_full[buf]));
                    tc_commit_pair(map_to_cta(smem_u32(&acc_full[buf]), 1));
                } else {
                    mbar_arrive(smem_u32(&acc_full[buf]));
                    mbar_arrive_cluster(map_to_cta(smem_u32(&acc_full[buf]), 1));
                }
            }
        }
    } else {
        // ---------------- epilogue (both CTAs, each for its own 128 rows) ----------------
        const int q = warp & 3, ch = (warp - 2) >> 2;
        int it = 0;
        bool ok = true;
        for (int item = cluster_id; item < p.n_items && ok; item += n_clusters, ++it) {
            const int pair = item % p.n_pairs, buf = it & 1;
            const long long row = (long long)(item / p.n_pairs) * (2 * kRows) + (long long)rank * kRows + q * 32 + lane;
            const bool in_range = row < p.rows;
            bool live_a = false, live_b = false;
            const int s_end = pair_ptr[pair + 1];
            for (int st = pair_ptr[pair]; st < s_end; ++st) {
                const int4 s = steps[st];
                live_a |= s.y >= 0;
                live_b |= s.z >= 0;
            }
            ok = mbar_wait_relaxed(smem_u32(&acc_full[buf]), (it >> 1) & 1, abort_flag, 8);
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t taddr = tmem + buf * kAccCols + ((uint32_t)(q * 32) << 16);
            if (p.swiglu) {
#pragma unroll 1
                for (int c0 = ch * 64; c0 < ch * 64 + 64; c0 += 32) {
                    const long long col0 = (long long)pair * 128 + c0;
                    if (p.gates == nullptr) block_epilogue_chunk<true, false>(p, taddr, row, in_range, col0, c0, live_a, live_b);
                    else block_epilogue_chunk<true, true>(p, taddr, row, in_range, col0, c0, live_a, live_b);
                }
            } else {
#pragma unroll 1
                for (int c0 = ch * 128; c0 < ch * 128 + 128; c0 += 32) {
                    const long long col0 = (long long)pair * 256 + c0;
                    block_epilogue_chunk<false, false>(p, taddr, row, in_range, col0, c0, c0 < 128 ? live_a : live_b, true);
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[buf]), 0));
        }
    }

    // neither CTA may leave (or free tensor memory) while its peer can still read its shared
    // memory or signal its barriers
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    cluster_sync_all();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

// Per-row symmetric int8 quantisation: scale[r] = max|x[r]| / 127, q = round(x / scale[r]).
// One CTA per row; the row is read twice (the second time from cache).
__global__ void __launch_bounds__(256)
quantize_rows_kernel(const __nv_bfloat16 *__restrict__ x, long long ldx, int cols, int8_t *__restrict__ q,
                     long long ldq, float *__restrict__ scale) {
    const long long row = blockIdx.x;
    const uint4 *src = reinterpret_cast<const uint4 *>(x + row * ldx);      // 8 values per load
    const int n8 = cols >> 3;
    float m = 0.f;
    for (int i = threadIdx.x; i < n8; i += blockDim.x) {
        const uint4 v = __ldg(src + i);
        const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __nv_bfloat162 h = __habs2(*reinterpret_cast<const __nv_bfloat162 *>(&ws[k]));
            m = fmaxf(m, fmaxf(__low2float(h), __high2float(h)));
        }
    }
    __shared__ float red[8];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    m = red[0];
#pragma unroll
    for (int k = 1; k < 8; ++k) m = fmaxf(m, red[k]);
    const float inv = m > 0.f ? 127.f / m : 0.f;
    if (threadIdx.x == 0) scale[row] = m / 127.f;
    uint2 *dst = reinterpret_cast<uint2 *>(q + row * ldq);
    for (int i = threadIdx.x; i < n8; i += blockDim.x) {
        const uint4 v = __ldg(src + i);
        const uint32_t ws[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[2] = {0u, 0u};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162 *>(&ws[k]);
            const int a = max(-127, min(127, __float2int_rn(__low2float(h) * inv)));
            const int b = max(-127, min(127, __float2int_rn(__high2float(h) * inv)));
            o[k >> 1] |= ((uint32_t)(a & 0xff) | ((uint32_t)(b & 0xff) << 8)) << ((k & 1) * 16);
        }
        dst[i] = make_uint2(o[0], o[1]);
    }
}

}  // namespace

extern "C" int mortar_linear_tc(const mortar_sched *w, const void *x, int64_t ldx, int64_t rows,
                                void *out, int64_t ld_out, const float *gates, int64_t ld_gates,
                                int32_t cluster_size, void *stream) {
    return linear_tc_impl<false>(w, x, ldx, rows, nullptr, out, ld_out, gates, ld_gates, cluster_size, stream);
}

extern "C" int mortar_linear_tc_i8(const mortar_sched *w, const void *xq, int64_t ldxq, const float *x_scale,
                                   int64_t rows, void *out, int64_t ld_out, const float *gates,
                                   int64_t ld_gates, int32_t cluster_size, void *stream) {
    return linear_tc_impl<true>(w, xq, ldxq, rows, x_scale, out, ld_out, gates, ld_gates, cluster_size, stream);
}

extern "C" int mortar_quantize_rows(const void *x, int64_t ldx, int64_t rows, int32_t cols, void *q,
                                    int64_t ldq, float *scale, void *stream) {
    if (!x || !q || !scale) return MORTAR_ERR_NULL;
    if (rows < 0 || cols <= 0 || (cols % 8) || ldx < cols || ldq < cols || rows > 0x7fffffffLL)
        return MORTAR_ERR_SHAPE;
    if (!aligned_to(x, 16) || (ldx % 8) || !aligned_to(q, 16) || (ldq % 16)) return MORTAR_ERR_ALIGN;
    if (rows == 0) return MORTAR_OK;
    quantize_rows_kernel<<<(unsigned)rows, 256, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const __nv_bfloat16 *>(x), ldx, cols, reinterpret_cast<int8_t *>(q), ldq, scale);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

extern "C" int mortar_linear_blocks_mode(int32_t mode) {
    if (mode < 0 || mode > 2) return MORTAR_ERR_SHAPE;
    return g_blocks_mode.exchange(mode, std::memory_order_relaxed);
}

extern "C" int mortar_linear_blocks(const mortar_blocks *w, const void *x, int64_t ldx, int64_t rows, void *out,
                                    int64_t ld_out, const float *gates, int64_t ld_gates, int32_t cluster_size,
                                    void *stream) {
    if (!w || !x || !out || !w->pair_ptr || (w->n_steps > 0 && (!w->steps || !w->data))) return MORTAR_ERR_NULL;
    if (w->n_pairs <= 0 || w->n_steps < 0 || w->out_features <= 0 || w->in_features <= 0 || rows < 0 ||
        (w->out_features % 16) || (w->in_features % 16))
        return MORTAR_ERR_SHAPE;
    const int n_out = w->swiglu ? w->out_features / 2 : w->out_features;
    // every output column belongs to a pair (SwiGLU: 128 hidden columns per pair, the last pair may be
    // padded; linear: 256 output columns per pair)
    if ((int64_t)w->n_pairs * (w->swiglu ? 128 : 256) < n_out) return MORTAR_ERR_SHAPE;
    if (ldx < w->in_features || ld_out < n_out) return MORTAR_ERR_SHAPE;
    if (!aligned_to(x, 16) || (ldx % 8) || !aligned_to(out, 16) || (ld_out % 8) || !aligned_to(w->data, 16) ||
        !aligned_to(w->steps, 16))
        return MORTAR_ERR_ALIGN;
    if (gates && (cluster_size <= 0 || !w->swiglu)) return MORTAR_ERR_SHAPE;
    if (rows == 0) return MORTAR_OK;
    // more than one block of rows: CTA pairs (never slower in measurements, a few percent faster where
    // most steps hold both blocks and the tensor pipe and shared-memory traffic bound the kernel)
    const int mode = g_blocks_mode.load(std::memory_order_relaxed);
    const bool pairs = mode == 2 || (mode == 0 && rows > kRows);
    const int item_rows = pairs ? 2 * kRows : kRows;
    const int64_t row_blocks = (rows + item_rows - 1) / item_rows;
    const int64_t n_items = row_blocks * w->n_pairs;
    if (n_items > 0x7fffffffLL || rows > 0x7fffffffLL - item_rows || w->n_blocks > (0x7fffffffLL >> 7))
        return MORTAR_ERR_CAPACITY;

    EncodeTiledFn encode;
    int rc = get_encode_fn(&encode);
    if (rc != MORTAR_OK) return rc;
    alignas(64) CUtensorMap tmap_x, tmap_w, tmap_wh;
    const cuuint32_t box[2] = {64, 128};
    const cuuint32_t box_half[2] = {64, 64};
    const cuuint32_t estride[2] = {1, 1};
    {
        const cuuint64_t gdim[2] = {(cuuint64_t)w->in_features, (cuuint64_t)rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)ldx * 2};
        if (encode(&tmap_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(x), gdim, gstride, box, estride,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            mortar_set_cuda_error("cuTensorMapEncodeTiled", "failed to encode the activation tensor map");
            return MORTAR_ERR_CUDA;
        }
    }
    {
        // the expanded blocks as one [n_blocks * 128][128] matrix (a matrix without blocks never loads from it)
        const cuuint64_t gdim[2] = {128, (cuuint64_t)(w->n_blocks > 0 ? w->n_blocks : 1) * 128};
        const cuuint64_t gstride[1] = {256};
        void *base = w->n_blocks > 0 ? const_cast<void *>(w->data) : const_cast<void *>(x);
        if (encode(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, gdim, gstride, box, estride,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            mortar_set_cuda_error("cuTensorMapEncodeTiled", "failed to encode the block tensor map");
            return MORTAR_ERR_CUDA;
        }
        // the same matrix in boxes of 64 block rows: the share of a block one CTA of a pair holds
        if (pairs && encode(&tmap_wh, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, gdim, gstride, box_half, estride,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            mortar_set_cuda_error("cuTensorMapEncodeTiled", "failed to encode the half-block tensor map");
            return MORTAR_ERR_CUDA;
        }
    }
    int dev = 0;
    MORTAR_CUDA_CHECK(cudaGetDevice(&dev));
    static int sm_count[64] = {0};
    if (dev < 0 || dev >= 64) return MORTAR_ERR_CAPACITY;
    int sms = 0;
    {
        std::lock_guard<std::mutex> lock(g_prefill_init_mutex);
        if (sm_count[dev] == 0) {
            int v = 0;
            MORTAR_CUDA_CHECK(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(prefill_blocks_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   kBkSmemBytes));
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(prefill_blocks_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   kB2SmemBytes));
            sm_count[dev] = v;
        }
        sms = sm_count[dev];
    }
    BlockParams p;
    p.pair_ptr = w->pair_ptr;
    p.steps = reinterpret_cast<const int4 *>(w->steps);
    p.n_pairs = w->n_pairs;
    p.n_steps = w->n_steps;
    p.n_items = (int)n_items;
    p.swiglu = w->swiglu;
    p.n_out = n_out;
    p.rows = rows;
    p.out = reinterpret_cast<__nv_bfloat16 *>(out);
    p.ld_out = ld_out;
    p.scale = __bfloat162float(__float2bfloat16_rn(w->scale));
    p.gates = gates;
    p.ld_gates = ld_gates;
    p.cluster_size = cluster_size > 0 ? cluster_size : 1;
    if (pairs) {
        const int64_t n_clusters = n_items < sms / 2 ? n_items : sms / 2;
        if (n_clusters < 1) return MORTAR_ERR_CAPACITY;
        prefill_blocks_pair_kernel<<<(unsigned)(2 * n_clusters), kBkThreads, kB2SmemBytes, (cudaStream_t)stream>>>(
            tmap_x, tmap_w, tmap_wh, p);
    } else {
        const unsigned grid = (unsigned)(n_items < sms ? n_items : sms);
        prefill_blocks_kernel<<<grid, kBkThreads, kBkSmemBytes, (cudaStream_t)stream>>>(tmap_x, tmap_w, p);
    }
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

extern "C" int mortar_mlp_prefill_blocks(const mortar_blocks *gate_up, const mortar_blocks *down, const void *x,
                                         int64_t ldx, int64_t rows, const float *gates, int64_t ld_gates,
                                         int32_t n_clusters, void *y, int64_t ldy, void *workspace,
                                         int64_t workspace_bytes, void *stream) {
    if (!gate_up || !down || !x || !y || !workspace) return MORTAR_ERR_NULL;
    if (!gate_up->swiglu || down->swiglu) return MORTAR_ERR_SHAPE;
    const int d_model = gate_up->in_features, d_ff = gate_up->out_features / 2;
    if (down->in_features != d_ff || down->out_features != d_model) return MORTAR_ERR_SHAPE;
    if (gates && (n_clusters <= 0 || d_ff % n_clusters)) return MORTAR_ERR_SHAPE;
    if (!aligned_to(workspace, 256)) return MORTAR_ERR_ALIGN;
    if (workspace_bytes < rows * (int64_t)d_ff * 2) return MORTAR_ERR_CAPACITY;
    int rc = mortar_linear_blocks(gate_up, x, ldx, rows, workspace, d_ff, gates, ld_gates,
                                  gates ? d_ff / n_clusters : 0, stream);
    if (rc != MORTAR_OK) return rc;
    return mortar_linear_blocks(down, workspace, d_ff, rows, y, ldy, nullptr, 0, 0, stream);
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

#ifdef MORTAR_PREFILL_TIMING
// Profiling builds only: copies (and clears) the 40 cycle counters.  Synchronises.
extern "C" int mortar_prefill_ticks(unsigned long long *out) {
    if (!out) return MORTAR_ERR_NULL;
    MORTAR_CUDA_CHECK(cudaMemcpyFromSymbol(out, g_prefill_ticks, sizeof(unsigned long long) * 40));
    static const unsigned long long zeros[40] = {0};
    MORTAR_CUDA_CHECK(cudaMemcpyToSymbol(g_prefill_ticks, zeros, sizeof(zeros)));
    return MORTAR_OK;
}
#endif

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
