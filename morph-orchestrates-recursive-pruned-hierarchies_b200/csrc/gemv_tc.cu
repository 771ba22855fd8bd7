// Decode GEMV for matrices carved in 128 x 128 blocks (the reference's carve granularity) and
// small batches, on the 5th-generation tensor cores: y = W x with the weights as the M side.
//
// `mortar_gemv` streams every kept block once per token step (fused_decode_step.py:1341-1459);
// per 64-byte tile the mma.sync path spends ~24 warp instructions (decode, fragment loads, index
// arithmetic, one MMA), which bounds it by instruction issue at 17% of the HBM rate.  Here a kept
// block is one unit of work: its 2-bit codes (4 KB) are bulk-copied into shared memory, eight
// warps expand them -- thread m owns output row m of the block -- and store them STRAIGHT INTO
// TENSOR MEMORY (tcgen05.st) as the A operand [128 rows x 128 inputs] of eight tcgen05.mma
// (M = 128, N = 16, K = 16), whose B operand is the block column's 4 KB slice of the activation
// operand (up to 16 columns = rows x exact bf16 planes).  No fragment loads, no per-tile index
// arithmetic, one MMA instruction per 16 x 128 codes; the decoded weights never touch shared memory.
//
// Persistent, one CTA of 14 warps per SM: warp 0 bulk-copy producer (12-stage ring of 8 KB: codes +
// activation slice), warp 1 MMA issue, warps 2..9 decode (lane quadrant = warp % 4, input half =
// (warp - 2) / 4), warps 10..13 epilogue.  Tensor memory: two accumulator sets of 32 columns (gate
// and up sums of one pair of block rows) and three decoded-block buffers of 64 columns.  Every
// mbarrier wait is bounded; on expiry the CTA records an error code and unwinds.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <mutex>
#include "common.h"
#include "decode.cuh"
#include "tc_common.cuh"

namespace {

constexpr int kStages = 12;
constexpr int kRawBytes = 8192;                      // 4 KB of row words + 4 KB of activation tiles
constexpr int kABufs = 3;
constexpr int kDecodeWarps = 8, kEpiWarps = 4;
constexpr int kThreads = 32 * (2 + kDecodeWarps + kEpiWarps);    // 448
constexpr int kTmemCols = 256;
constexpr int kAccCol = 0;                           // 2 x 32 accumulator columns
constexpr int kACol = 64;                            // 3 x 64 columns of decoded weights
constexpr int kSmemBytes = kStages * kRawBytes + (2 * kStages + 2 * kABufs + 4) * 8 + 1024;
constexpr uint32_t kWaitLimit = 1u << 22;

__device__ int g_gemv_tc_error;

#ifdef MORTAR_GEMV_TIMING
__device__ unsigned long long g_gemv_ticks[24];
#define GT_DECL long long tk[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long tprev = clock64()
#define GT_ACC(i) do { const long long tn_ = clock64(); tk[i] += tn_ - tprev; tprev = tn_; } while (0)
#define GT_PUT(base, cond) do { if ((cond) && blockIdx.x == 0) for (int i_ = 0; i_ < 8; ++i_) \
        atomicAdd(&g_gemv_ticks[(base) + i_], (unsigned long long)tk[i_]); } while (0)
#else
#define GT_DECL
#define GT_ACC(i)
#define GT_PUT(base, cond)
#endif

struct GemvTcParams {
    const uint8_t *words;        // [n_blocks][128 rows][8] permuted row words (32 bytes per row)
    const uint8_t *xb;           // activation operand [in/16][512 B]
    const int *blk_ptr;          // [block rows + 1]
    const int *blk_col;          // [n_blocks]
    const int *items;            // [n_items] first block row of every item, largest first
    int n_items;
    int half_rows;               // swiglu: block rows of the gate half (the up row of item g is g + half_rows)
    int swiglu;
    int rows, n_planes;          // accumulator column = plane * rows + row
    float scale;
    void *out;
    int out_mode, n_out_planes;
    long long out_plane_stride, ld_out;
};

// The blocks of this CTA's items in order: item (stride gridDim.x), its one or two block rows, their blocks.
struct BlockWalk {
    int item, sub, b, b_end;
    __device__ __forceinline__ bool valid(const GemvTcParams &p) const { return item < p.n_items; }
    __device__ __forceinline__ void settle(const GemvTcParams &p) {
        // move forward to the next (item, sub) that has a block
        while (item < p.n_items) {
            const int nsub = p.swiglu ? 2 : 1;
            while (sub < nsub) {
                const int brow = __ldg(p.items + item) + sub * p.half_rows;
                b = __ldg(p.blk_ptr + brow);
                b_end = __ldg(p.blk_ptr + brow + 1);
                if (b < b_end) return;
                ++sub;
            }
            item += gridDim.x;
            sub = 0;
        }
    }
    __device__ __forceinline__ void start(const GemvTcParams &p) { item = blockIdx.x; sub = 0; b = b_end = 0; settle(p); }
    __device__ __forceinline__ void next(const GemvTcParams &p) {
        if (++b < b_end) return;
        ++sub;
        settle(p);
    }
};

__device__ __forceinline__ void st32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};\n"
        "tcgen05.wait::st.sync.aligned;\n"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}

__device__ __forceinline__ void ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
          "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}

// A from tensor memory, B from shared memory.
__device__ __forceinline__ void mma_a_tmem(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(accumulate));
}

template <bool ACC>
__device__ __forceinline__ void mma_a_tmem_lit(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.eq.u32 p, %4, 1;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n"
        ::"r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc), "n"(ACC ? 1 : 0));
}

// One block: the polls of the NEXT block's two barriers and this block's eight MMAs (A operand 8
// tensor-memory columns apart, B descriptor 512 bytes apart) as one instruction sequence, so the
// polls' results are first read after the MMAs have issued.  Returns whether both polled phases
// had completed.
template <bool FIRST_ACC>
__device__ __forceinline__ bool poll2_mma8(uint32_t bar1, uint32_t parity1, uint32_t bar2, uint32_t parity2,
                                           uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc) {
    uint32_t ready;
#define MORTAR_GEMV_NEXT_MMA "add.u32 aa, aa, 8;\n add.u64 db, db, 32;\n tcgen05.mma.cta_group::1.kind::f16 [%5], [aa], db, %8, p1;\n"
    asm volatile(
        "{\n.reg .pred q1, q2, p0, p1;\n.reg .b64 db;\n.reg .b32 aa;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 q1, [%1], %2;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 q2, [%3], %4;\n"
        "setp.eq.u32 p0, %9, 1;\n setp.eq.u32 p1, 1, 1;\n"
        "mov.b64 db, %7;\n mov.b32 aa, %6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%5], [aa], db, %8, p0;\n"
        MORTAR_GEMV_NEXT_MMA MORTAR_GEMV_NEXT_MMA MORTAR_GEMV_NEXT_MMA MORTAR_GEMV_NEXT_MMA
        MORTAR_GEMV_NEXT_MMA MORTAR_GEMV_NEXT_MMA MORTAR_GEMV_NEXT_MMA
        "and.pred q1, q1, q2;\n selp.b32 %0, 1, 0, q1;\n}\n"
        : "=r"(ready)
        : "r"(bar1), "r"(parity1), "r"(bar2), "r"(parity2), "r"(d_tmem), "r"(a_tmem), "l"(bdesc), "r"(idesc),
          "n"(FIRST_ACC ? 1 : 0)
        : "memory");
#undef MORTAR_GEMV_NEXT_MMA
    return ready != 0;
}

__device__ __forceinline__ void arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(bar) : "memory");
}

__global__ void __launch_bounds__(kThreads, 1) gemv_tc_kernel(const GemvTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *stages = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *raw_full = reinterpret_cast<uint64_t *>(stages + kStages * kRawBytes), *raw_empty = raw_full + kStages;
    uint64_t *a_full = raw_empty + kStages, *a_empty = a_full + kABufs;
    uint64_t *acc_full = a_empty + kABufs, *acc_empty = acc_full + 2;
    __shared__ uint32_t tmem_base_s;
    __shared__ int abort_s;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        abort_s = 0;
        for (int s = 0; s < kStages; ++s) {
            tc::mbar_init(tc::smem_u32(&raw_full[s]), 1);
            tc::mbar_init(tc::smem_u32(&raw_empty[s]), kDecodeWarps + 1);   // the decoders and the MMAs' commit
        }
        for (int s = 0; s < kABufs; ++s) { tc::mbar_init(tc::smem_u32(&a_full[s]), kDecodeWarps); tc::mbar_init(tc::smem_u32(&a_empty[s]), 1); }
        for (int s = 0; s < 2; ++s) { tc::mbar_init(tc::smem_u32(&acc_full[s]), 1); tc::mbar_init(tc::smem_u32(&acc_empty[s]), kEpiWarps); }
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

    // The producer and the MMA role are one thread each.  What such a thread spends between the
    // MMAs of two blocks (polls, commits, address arithmetic, the walk over the block lists) is
    // time the tensor pipe drains, because its queue holds only about four MMAs: so the poll of
    // the next block's barrier and the loads the next block needs are issued before the work of
    // the current one, the accumulate flag is a compile-time constant, and nothing is recomputed
    // per MMA that is fixed per block.
    if (warp == 0) {
        // ---------------- producer: codes and activation slice of every block ----------------
        if (lane == 0) {
            const uint32_t full0 = tc::smem_u32(&raw_full[0]), empty0 = tc::smem_u32(&raw_empty[0]), stage0 = tc::smem_u32(stages);
            // w walks the blocks, wl runs two blocks ahead of it: a block's column index (a load from
            // global memory the activation slice's address depends on) is requested two blocks early
            BlockWalk w, wl;
            w.start(p);
            wl = w;
            int c0 = 0, c1 = 0;
            if (wl.valid(p)) { c0 = __ldg(p.blk_col + wl.b); wl.next(p); }
            if (wl.valid(p)) { c1 = __ldg(p.blk_col + wl.b); wl.next(p); }
            uint32_t n = 0u;
            bool ok = true;
            bool ready = tc::mbar_try_wait(empty0, 1u);
            auto load_block = [&](int b, int col) {
                const uint32_t s = n % kStages;
                if (!ready) ok = tc::mbar_wait(empty0 + s * 8u, ((n / kStages) & 1u) ^ 1u, abort_flag, &g_gemv_tc_error, 1, kWaitLimit);
                if (!ok) return;
                const uint32_t nx = n + 1u;
                ready = tc::mbar_try_wait(empty0 + (nx % kStages) * 8u, ((nx / kStages) & 1u) ^ 1u);
                const uint32_t bar = full0 + s * 8u;
                const uint32_t dst = stage0 + s * (uint32_t)kRawBytes;
                tc::mbar_arrive_expect_tx(bar, kRawBytes);
                const uint8_t *src_w = p.words + (size_t)b * 4096;
                const uint8_t *src_x = p.xb + (size_t)col * 4096;
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                             ::"r"(dst), "l"(src_w), "r"(4096), "r"(bar) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                             ::"r"(dst + 4096), "l"(src_x), "r"(4096), "r"(bar) : "memory");
                ++n;
            };
            while (w.valid(p) && ok) {
                load_block(w.b, c0);
                w.next(p);
                if (wl.valid(p)) { c0 = __ldg(p.blk_col + wl.b); wl.next(p); }
                if (!w.valid(p) || !ok) break;
                load_block(w.b, c1);
                w.next(p);
                if (wl.valid(p)) { c1 = __ldg(p.blk_col + wl.b); wl.next(p); }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issue ----------------
        // kind::f16, D fp32 (bit 4), A and B bf16 (bits 7, 10), both K-major, N = 16 (>> 3 at bit 17), M = 128 (>> 4 at bit 24)
        constexpr uint32_t kIdesc = (1u << 4) | (1u << 7) | (1u << 10) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
        if (lane == 0) {
            // activation tile kk of a block column: [16 columns x 16 inputs], K-major, no swizzle, 512 bytes
            // apart; only the address field of the descriptor changes between MMAs and stages
            const uint64_t bd0 = tc::make_smem_desc(tc::smem_u32(stages) + 4096, 128, 256, 0);
            const uint32_t afull0 = tc::smem_u32(&a_full[0]), aempty0 = tc::smem_u32(&a_empty[0]);
            const uint32_t rfull0 = tc::smem_u32(&raw_full[0]), rempty0 = tc::smem_u32(&raw_empty[0]);
            BlockWalk w;
            w.start(p);
            int n = 0, it = -1, cur_item = -1, cur_sub = -1;
            uint32_t ab = 0u, ab_phase = 0u;                         // tensor-memory operand buffer of block n and its phase
            bool ok = true;
            // both barriers of the next block (its stage: the activation slice; its operand buffer: the
            // decoded weights) are polled a block ahead
            bool ready = tc::mbar_try_wait(rfull0, 0u) && tc::mbar_try_wait(afull0, 0u);
            GT_DECL;
            while (w.valid(p)) {
                GT_ACC(0);
                if (w.item != cur_item) {
                    // the previous item is complete once its MMAs retire
                    if (cur_item >= 0) tc::commit(tc::smem_u32(&acc_full[it & 1]));
                    cur_item = w.item; cur_sub = -1; ++it;
                    if (!tc::mbar_try_wait(tc::smem_u32(&acc_empty[it & 1]), ((it >> 1) & 1) ^ 1u))
                        ok = tc::mbar_wait(tc::smem_u32(&acc_empty[it & 1]), ((it >> 1) & 1) ^ 1u, abort_flag, &g_gemv_tc_error, 9, kWaitLimit);
                    if (!ok) break;
                }
                const bool first = w.sub != cur_sub;                 // first block of this block row: overwrite
                cur_sub = w.sub;
                const uint32_t acc = tmem + kAccCol + (uint32_t)(it & 1) * 32u + (uint32_t)w.sub * 16u;
                const uint32_t s = (uint32_t)n % kStages;
                w.next(p);                                           // the walk's loads run under this block's MMAs
                GT_ACC(1);
                if (!ready)
                    ok = tc::mbar_wait(rfull0 + s * 8u, ((uint32_t)n / kStages) & 1u, abort_flag, &g_gemv_tc_error, 2, kWaitLimit) &&
                         tc::mbar_wait(afull0 + ab * 8u, ab_phase, abort_flag, &g_gemv_tc_error, 3, kWaitLimit);
                if (!ok) break;
                GT_ACC(2);
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t ab_next = ab == kABufs - 1 ? 0u : ab + 1u, phase_next = ab == kABufs - 1 ? ab_phase ^ 1u : ab_phase;
                const uint32_t nx = (uint32_t)n + 1u;
                const uint32_t a0 = tmem + kACol + ab * 64u;
                const uint64_t bd = bd0 + (uint64_t)(s * (uint32_t)(kRawBytes >> 4));
                const uint32_t rbar = rfull0 + (nx % kStages) * 8u, rpar = (nx / kStages) & 1u, abar = afull0 + ab_next * 8u;
                ready = first ? poll2_mma8<false>(rbar, rpar, abar, phase_next, acc, a0, bd, kIdesc)
                              : poll2_mma8<true>(rbar, rpar, abar, phase_next, acc, a0, bd, kIdesc);
                GT_ACC(3);
                tc::commit(aempty0 + ab * 8u);
                tc::commit(rempty0 + s * 8u);
                GT_ACC(4);
                ab = ab_next;
                ab_phase = phase_next;
                ++n;
            }
            if (ok && cur_item >= 0) tc::commit(tc::smem_u32(&acc_full[it & 1]));
            GT_PUT(8, true);
        }
    } else if (warp < 2 + kDecodeWarps) {
        // ---------------- decode: codes -> bf16 rows of the A operand in tensor memory ----------------
        const int quad = warp & 3, kh = (warp - 2) >> 2;              // lane quadrant (fixed by the warp id), input half
        const int m = quad * 32 + lane;                               // output row of the block
        BlockWalk w;
        int n = 0;
        GT_DECL;
        for (w.start(p); w.valid(p); w.next(p), ++n) {
            const int s = n % kStages, ab = n % kABufs;
            GT_ACC(0);
            if (!tc::mbar_wait(tc::smem_u32(&raw_full[s]), (n / kStages) & 1, abort_flag, &g_gemv_tc_error, 4, kWaitLimit)) break;
            GT_ACC(1);
            const uint4 wv = *reinterpret_cast<const uint4 *>(stages + s * kRawBytes + m * 32 + kh * 16);
            const uint32_t ws[4] = {wv.x, wv.y, wv.z, wv.w};
            uint32_t r[32];
#pragma unroll
            for (int tcl = 0; tcl < 4; ++tcl)
#pragma unroll
                for (int q = 0; q < 8; ++q) r[tcl * 8 + q] = mortar_decode_pair(ws[tcl], q);
            GT_ACC(2);
            if (!tc::mbar_wait(tc::smem_u32(&a_empty[ab]), ((n / kABufs) & 1) ^ 1u, abort_flag, &g_gemv_tc_error, 5, kWaitLimit)) break;
            GT_ACC(3);
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            st32(tmem + kACol + ab * 64 + kh * 32 + ((uint32_t)(quad * 32) << 16), r);
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                arrive(tc::smem_u32(&a_full[ab]));
                arrive(tc::smem_u32(&raw_empty[s]));
            }
            GT_ACC(4);
        }
        GT_PUT(16, warp == 2 && lane == 0);
    } else {
        // ---------------- epilogue: one item = 128 output features ----------------
        const int quad = warp & 3;
        const int m = quad * 32 + lane;
        const int nsub = p.swiglu ? 2 : 1;
        int it = 0;
        for (int item = blockIdx.x; item < p.n_items; item += gridDim.x) {
            const int brow0 = __ldg(p.items + item);
            bool live[2] = {false, false};
            bool any = false;
            for (int sub = 0; sub < nsub; ++sub) {
                const int brow = brow0 + sub * p.half_rows;
                live[sub] = __ldg(p.blk_ptr + brow + 1) > __ldg(p.blk_ptr + brow);
                any |= live[sub];
            }
            uint32_t a[32];
            if (any) {                                               // an item without blocks never reaches the MMA warp
                if (!tc::mbar_wait(tc::smem_u32(&acc_full[it & 1]), (it >> 1) & 1, abort_flag, &g_gemv_tc_error, 8, 1u << 26)) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                ld32(tmem + kAccCol + (it & 1) * 32 + ((uint32_t)(quad * 32) << 16), a);
                asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
                __syncwarp();
                if (lane == 0) arrive(tc::smem_u32(&acc_empty[it & 1]));
                ++it;
            }
            const long long f = (long long)brow0 * 128 + m;          // output feature (hidden feature for SwiGLU)
            for (int r = 0; r < p.rows; ++r) {
                float sa = 0.f, sb = 0.f;
                for (int pl = 0; pl < p.n_planes; ++pl) {
                    const int c = pl * p.rows + r;
                    // dynamic register indexing would spill: select the column with a compile-time loop
#pragma unroll
                    for (int k = 0; k < 16; ++k) {
                        if (k == c) { sa += __uint_as_float(a[k]); sb += __uint_as_float(a[16 + k]); }
                    }
                }
                float v;
                if (p.swiglu) {
                    const float gv = live[0] ? p.scale * sa : 0.f, uv = live[1] ? p.scale * sb : 0.f;
                    v = gv * (1.f / (1.f + expf(-gv))) * uv;
                } else {
                    v = live[0] ? p.scale * sa : 0.f;
                }
                if (p.out_mode == MORTAR_OUT_F32) {
                    reinterpret_cast<float *>(p.out)[r * p.ld_out + f] = v;
                } else if (p.out_mode == MORTAR_OUT_BF16) {
                    reinterpret_cast<__nv_bfloat16 *>(p.out)[r * p.ld_out + f] = __float2bfloat16_rn(v);
                } else {                                             // exact bf16 planes for the next product
                    __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(p.out) + r * p.ld_out + f;
                    for (int pl = 0; pl < p.n_out_planes; ++pl) {
                        const __nv_bfloat16 h = __float2bfloat16_rn(v);
                        o[pl * p.out_plane_stride] = h;
                        v -= __bfloat162float(h);
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (warp == 1)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(kTmemCols) : "memory");
}

// planes [P][rows][ld] bf16 -> activation operand: per 16 inputs one [16 columns x 16 inputs] tile,
// K-major without swizzle (8 x 16-byte core matrices: column group, input half), column = plane * rows + row.
__global__ void gemv_xprep_kernel(const __nv_bfloat16 *planes, int n_planes, long long plane_stride, long long ld,
                                  int rows, int in_features, uint8_t *xb) {
    const int tile = blockIdx.x;                         // 16 inputs
    const int chunk = threadIdx.x;                       // 32 chunks of 16 bytes
    const int n = (chunk >> 4) * 8 + (chunk & 7), kh = (chunk >> 3) & 1;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (n < n_planes * rows) {
        const int pl = n / rows, r = n - pl * rows;
        v = *reinterpret_cast<const uint4 *>(planes + pl * plane_stride + r * ld + tile * 16 + kh * 8);
    }
    *reinterpret_cast<uint4 *>(xb + (size_t)tile * 512 + (chunk >> 4) * 256 + kh * 128 + (chunk & 7) * 16) = v;
}

// The same operand from the fp32 result of a gate/up product [rows][2 d_ff] (gate columns, then up
// columns): h = silu(gate) * up, split into n_planes exact bf16 planes on the way -- the SwiGLU of a
// gate/up matrix whose d_ff is not a multiple of 128, where gate and up block rows do not pair up.
__global__ void gemv_xprep_swiglu_kernel(const float *gu, long long ld, int rows, int d_ff, int n_planes, uint8_t *xb) {
    const int tile = blockIdx.x;
    const int chunk = threadIdx.x;
    const int n = (chunk >> 4) * 8 + (chunk & 7), kh = (chunk >> 3) & 1;
    uint32_t packed[4] = {0u, 0u, 0u, 0u};
    if (n < n_planes * rows) {
        const int pl = n / rows, r = n - pl * rows;
        const float *g = gu + r * ld + tile * 16 + kh * 8, *u = g + d_ff;
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
            float v[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float gv = g[k + e];
                v[e] = gv * (1.f / (1.f + expf(-gv))) * u[k + e];
                for (int q = 0; q < pl; ++q) v[e] -= __bfloat162float(__float2bfloat16_rn(v[e]));   // peel the planes before this one
            }
            const __nv_bfloat162 h = __floats2bfloat162_rn(v[0], v[1]);
            packed[k >> 1] = *reinterpret_cast<const uint32_t *>(&h);
        }
    }
    *reinterpret_cast<uint4 *>(xb + (size_t)tile * 512 + (chunk >> 4) * 256 + kh * 128 + (chunk & 7) * 16) =
        make_uint4(packed[0], packed[1], packed[2], packed[3]);
}

std::mutex g_gemv_tc_mutex;

}  // namespace

extern "C" int mortar_gemv_xprep(const void *planes, int32_t n_planes, int64_t plane_stride, int64_t ld_planes,
                                 int64_t rows, int32_t in_features, void *xb, void *stream) {
    if (!planes || !xb) return MORTAR_ERR_NULL;
    if (n_planes < 1 || rows < 1 || n_planes * rows > 16 || in_features <= 0 || (in_features % 16) ||
        ld_planes < in_features)
        return MORTAR_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(planes) % 16) || (ld_planes % 8) || (plane_stride % 8) ||
        (reinterpret_cast<uintptr_t>(xb) % 128))
        return MORTAR_ERR_ALIGN;
    gemv_xprep_kernel<<<(unsigned)(in_features / 16), 32, 0, (cudaStream_t)stream>>>(
        reinterpret_cast<const __nv_bfloat16 *>(planes), n_planes, plane_stride, ld_planes, (int)rows, in_features,
        reinterpret_cast<uint8_t *>(xb));
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

extern "C" int mortar_gemv_xprep_swiglu(const float *gate_up, int64_t ld, int64_t rows, int32_t d_ff, int32_t n_planes,
                                        void *xb, void *stream) {
    if (!gate_up || !xb) return MORTAR_ERR_NULL;
    if (n_planes < 1 || n_planes > 3 || rows < 1 || n_planes * rows > 16 || d_ff <= 0 || (d_ff % 16) || ld < 2 * (int64_t)d_ff)
        return MORTAR_ERR_SHAPE;
    if (reinterpret_cast<uintptr_t>(xb) % 128) return MORTAR_ERR_ALIGN;
    gemv_xprep_swiglu_kernel<<<(unsigned)(d_ff / 16), 32, 0, (cudaStream_t)stream>>>(gate_up, ld, (int)rows, d_ff, n_planes,
                                                                                   reinterpret_cast<uint8_t *>(xb));
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

extern "C" int mortar_gemv_blocks(const mortar_gemv_pack *w, const void *xb, int64_t rows, int32_t n_planes,
                                  void *out, int32_t out_mode, int32_t n_out_planes, int64_t out_plane_stride,
                                  int64_t ld_out, void *stream) {
    if (!w || !xb || !out || !w->row_words || !w->blk_ptr || !w->blk_col || !w->items) return MORTAR_ERR_NULL;
    if (w->n_items < 0 || w->out_features <= 0 || w->in_features <= 0 || (w->out_features % 128) ||
        (w->in_features % 128) || rows < 1 || n_planes < 1 || rows * n_planes > 16)
        return MORTAR_ERR_SHAPE;
    const int n_out = w->swiglu ? w->out_features / 2 : w->out_features;
    if (w->swiglu && (n_out % 128)) return MORTAR_ERR_SHAPE;
    if (ld_out < n_out) return MORTAR_ERR_SHAPE;
    if (out_mode != MORTAR_OUT_F32 && out_mode != MORTAR_OUT_BF16 && out_mode != MORTAR_OUT_PLANES) return MORTAR_ERR_DTYPE;
    if (out_mode == MORTAR_OUT_PLANES && (n_out_planes < 1 || n_out_planes > 3)) return MORTAR_ERR_DTYPE;
    if ((reinterpret_cast<uintptr_t>(w->row_words) % 16) || (reinterpret_cast<uintptr_t>(xb) % 128)) return MORTAR_ERR_ALIGN;
    if (w->n_items == 0) return MORTAR_OK;
    int dev = 0;
    MORTAR_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MORTAR_ERR_CAPACITY;
    static int sm_count[64] = {0};
    int sms = 0;
    {
        std::lock_guard<std::mutex> lock(g_gemv_tc_mutex);
        if (sm_count[dev] == 0) {
            int v = 0;
            MORTAR_CUDA_CHECK(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(gemv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes));
            sm_count[dev] = v;
        }
        sms = sm_count[dev];
    }
    GemvTcParams p;
    p.words = reinterpret_cast<const uint8_t *>(w->row_words);
    p.xb = reinterpret_cast<const uint8_t *>(xb);
    p.blk_ptr = w->blk_ptr; p.blk_col = w->blk_col; p.items = w->items;
    p.n_items = w->n_items;
    p.half_rows = w->swiglu ? n_out / 128 : 0;
    p.swiglu = w->swiglu;
    p.rows = (int)rows; p.n_planes = n_planes;
    p.scale = w->scale;
    p.out = out; p.out_mode = out_mode; p.n_out_planes = n_out_planes;
    p.out_plane_stride = out_plane_stride; p.ld_out = ld_out;
    const unsigned grid = (unsigned)(w->n_items < sms ? w->n_items : sms);
    gemv_tc_kernel<<<grid, kThreads, kSmemBytes, (cudaStream_t)stream>>>(p);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

#ifdef MORTAR_GEMV_TIMING
extern "C" int mortar_gemv_ticks(unsigned long long *out) {
    MORTAR_CUDA_CHECK(cudaMemcpyFromSymbol(out, g_gemv_ticks, sizeof(unsigned long long) * 24));
    static const unsigned long long zeros[24] = {0};
    MORTAR_CUDA_CHECK(cudaMemcpyToSymbol(g_gemv_ticks, zeros, sizeof(zeros)));
    return MORTAR_OK;
}
#endif

extern "C" int mortar_gemv_blocks_error(int32_t *code, int32_t reset) {
    if (!code) return MORTAR_ERR_NULL;
    int v = 0;
    MORTAR_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_gemv_tc_error, sizeof(int)));
    *code = v;
    if (reset && v != 0) {
        const int zero = 0;
        MORTAR_CUDA_CHECK(cudaMemcpyToSymbol(g_gemv_tc_error, &zero, sizeof(int)));
    }
    return MORTAR_OK;
}
