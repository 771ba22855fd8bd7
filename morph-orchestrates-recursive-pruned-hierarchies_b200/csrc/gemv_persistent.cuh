// Persistent small-batch kernel over the 8-tile-group layout (included by stream_kernels.cu).
//
// For at most 8 MMA columns of activations (up to 8 bf16 rows, or 2 fp32 rows as 3 exact planes
// folded into the columns) against a matrix far larger than L2, the work per weight byte is so
// small that everything besides the weight stream has to be taken off the critical path:
//   * one CTA of 24 warps per SM (85 registers per thread: measured faster than 32 warps at 64
//     or 16 at 128), resident for the whole launch; the CTA's share of the matrix
//     is a contiguous range of units balanced by group count (found by a parallel search of the
//     row-pointer prefix sums, no atomics, no scratch memory);
//   * the activations are staged ONCE per CTA into shared memory, laid out so that a lane's
//     whole B fragment is one conflict-free 64-bit load;
//   * four slots of 5 consumer warps each walk the CTA's units; every slot owns a ring of stages
//     that its own producer warp (warps 20..23) fills with bulk asynchronous copies (mbarrier
//     completion), so the weight bytes of the next chunks are in flight while the current one
//     is decoded and multiplied, and nothing a consumer does can delay a refill;
//   * partial sums of the 5 warps of a slot meet in shared memory and are added in warp order
//     by one of them (taking turns, unit by unit), which also runs the epilogue.
// The epilogue is the one of the row-block kernel, so results follow the same rounding rules.
#pragma once

constexpr int kPsWarps = 24;            // warps per CTA
constexpr int kPsSlots = 4;             // units in flight per CTA
constexpr int kPsSlotWarps = 5;         // consumer warps per slot; warp 20 + slot is the slot's producer
constexpr int kPsConsumers = kPsSlots * kPsSlotWarps * 32;
constexpr int kPsStages = 3;            // ring depth per slot
constexpr int kPsChunk = 16;            // groups per stage (8 KB of codes + 256 B of column indices)
constexpr int kPsMaxSmem = 227 * 1024;
constexpr int kPsTabUnits = 64;         // units of a CTA whose row pointers are cached in shared memory

struct PsLayout {
    int stages, cols, bars, red, fold, misc, tab, x, total; // byte offsets into dynamic shared memory
    int x_pitch;                                            // bytes between activation rows
};

__host__ __device__ inline PsLayout ps_layout(int C, int vrows, bool swiglu) {
    PsLayout L;
    int off = 0;
    L.stages = off; off += kPsSlots * kPsStages * kPsChunk * 512;
    L.cols = off;   off += kPsSlots * kPsStages * kPsChunk * 16;
    L.bars = off;   off += kPsSlots * 2 * kPsStages * 8;
    L.red = off;    off += 2 * kPsSlots * kPsSlotWarps * (swiglu ? 2 : 1) * 4 * 32 * 4;   // two buffers, by unit parity
    L.fold = off;   off += kPsSlots * 2 * 16 * 9 * 4;
    L.misc = off;   off += 16;
    L.tab = off;    off += kPsTabUnits * 2 * 2 * 4;          // (first group, group count) of both tile rows
    off = (off + 127) / 128 * 128;
    // rows 32 bytes apart modulo 128, so the 16 lanes of a half-warp (4 rows x 4 lane pairs of
    // 8 bytes) cover all 32 banks once
    L.x_pitch = C * 32;
    while (L.x_pitch % 128 != 32) L.x_pitch += 32;
    L.x = off;      off += vrows * L.x_pitch;
    L.total = off;
    return L;
}

// Walks the chunks (at most kPsChunk groups of one tile row) of the units u0, u0+step, ... < u1
// in the order the consumers use them; tile rows without groups are skipped.
template <bool SWIGLU>
struct PsChunkWalk {
    int u, u1, a, cc, gbeg, len;
    const int *grp_ptr;
    int units;
    __device__ __forceinline__ void load_row() {
        const int trow = u + a * units;
        gbeg = __ldg(grp_ptr + trow);
        len = __ldg(grp_ptr + trow + 1) - gbeg;
    }
    __device__ __forceinline__ void init(const int *gp, int n_units, int u0, int uend) {
        grp_ptr = gp; units = n_units; u = u0; u1 = uend; a = 0; cc = 0; gbeg = 0; len = 0;
        if (u < u1) { load_row(); settle(); }
    }
    // moves forward until (u, a, cc) names an existing chunk or the units are used up
    __device__ __forceinline__ void settle() {
        while (u < u1 && cc * kPsChunk >= len) {
            cc = 0;
            if (SWIGLU && a == 0) a = 1;
            else { a = 0; u += kPsSlots; }
            if (u < u1) load_row();
        }
    }
    __device__ __forceinline__ bool valid() const { return u < u1; }
    __device__ __forceinline__ void get(int &g0, int &ng) const {
        g0 = gbeg + cc * kPsChunk;
        ng = min(kPsChunk, len - cc * kPsChunk);
    }
    __device__ __forceinline__ void next() { ++cc; settle(); }
};

__device__ __forceinline__ void ps_slot_sync(int slot) {
    asm volatile("bar.sync %0, %1;" ::"r"(slot + 1), "r"(kPsSlotWarps * 32) : "memory");
}

// Bounded wait that sleeps between polls, so waiting warps leave the issue slots to the others.
__device__ __forceinline__ bool ps_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kBulkWaitLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
        __nanosleep(40);
    }
    return false;
}

// One 8-tile group from shared memory against the staged activations.  `xs_lane` is the shared
// address of this lane's fragment of tile column 0; a tile column is 32 bytes further.
template <bool CHECK>
__device__ __forceinline__ void ps_group(float (&acc)[4], uint32_t codes_a, uint32_t cols_a,
                                         uint32_t xs_lane) {
    uint4 cw;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(cw.x), "=r"(cw.y), "=r"(cw.z), "=r"(cw.w) : "r"(codes_a));
    const uint32_t cws[4] = {cw.x, cw.y, cw.z, cw.w};
    uint32_t col[8], b0[8], b1[8];
#pragma unroll
    for (int s = 0; s < 8; ++s) asm volatile("ld.shared.u16 %0, [%1];" : "=r"(col[s]) : "r"(cols_a + 2u * s));
#pragma unroll
    for (int s = 0; s < 8; ++s)
        if (!CHECK || col[s] != 0xffffu)                             // padding slots end a row
            asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(b0[s]), "=r"(b1[s]) : "r"(xs_lane + col[s] * 32u));
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        if (!CHECK || col[s] != 0xffffu) {
            uint32_t af[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) af[i] = mortar_decode_pair(cws[s >> 1], (s & 1) * 4 + i);
            mma_16816(acc, af, b0[s], b1[s]);
        }
    }
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kPsWarps * 32, 1)
gemv_persistent_kernel(const LinearParams p) {
    constexpr int NACC = SWIGLU ? 2 : 1;
    constexpr int S = kPsStages, CG = kPsChunk;
    extern __shared__ __align__(128) unsigned char ps_smem[];
    const int vrows = (int)p.rows;                                   // MMA columns in use (<= 8)
    const PsLayout L = ps_layout(p.C, vrows, SWIGLU);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned long long *bars = reinterpret_cast<unsigned long long *>(ps_smem + L.bars);
    int *misc = reinterpret_cast<int *>(ps_smem + L.misc);   // [0], [1]: unit range of this CTA, [2]: a wait gave up

    if (tid < kPsSlots * 2 * S) {                                    // full[S] then empty[S] per slot
        const bool is_full = (tid % (2 * S)) < S;
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bars + tid)),
                     "r"(is_full ? 1 : kPsSlotWarps));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (tid == 0) { misc[0] = p.units; misc[1] = p.units; misc[2] = 0; }
    __syncthreads();

    // ---- this CTA's units: those whose first group lies in its share of the group count ----
    {
        const int *gp = p.grp_ptr;
        const long long base = SWIGLU ? (long long)__ldg(gp + p.units) : 0;
        const long long total = SWIGLU ? (long long)__ldg(gp + 2 * p.units) : (long long)__ldg(gp + p.units);
        const long long t_lo = total * blockIdx.x / gridDim.x, t_hi = total * (blockIdx.x + 1) / gridDim.x;
        auto cost_before = [&](int u) -> long long {          // groups of units [0, u)
            return SWIGLU ? (long long)__ldg(gp + u) + (long long)__ldg(gp + p.units + u) - base
                          : (long long)__ldg(gp + u);
        };
        for (int u = tid; u < p.units; u += kPsWarps * 32) {
            const long long c1 = cost_before(u);
            const long long c0 = u > 0 ? cost_before(u - 1) : -1;
            if (c1 >= t_lo && c0 < t_lo) misc[0] = u;
            // the last share keeps the preset upper end (all remaining units)
            if (blockIdx.x != gridDim.x - 1 && c1 >= t_hi && c0 < t_hi) misc[1] = u;
        }
    }
    __syncthreads();
    const int u_lo = misc[0], u_hi = misc[1];
    // row pointers of this CTA's first kPsTabUnits units -> shared memory (a tile row starts every
    // few hundred cycles per slot; a dependent global load there would be on the critical path)
    int *tab = reinterpret_cast<int *>(ps_smem + L.tab);
    for (int e = tid; e < kPsTabUnits * NACC; e += kPsWarps * 32) {
        const int ul = e / NACC, a = e % NACC;
        if (u_lo + ul < u_hi) {
            const int trow = u_lo + ul + a * p.units;
            const int gbeg = __ldg(p.grp_ptr + trow);
            tab[(ul * 2 + a) * 2] = gbeg;
            tab[(ul * 2 + a) * 2 + 1] = __ldg(p.grp_ptr + trow + 1) - gbeg;
        }
    }
    __syncthreads();
    auto row_info = [&](int u, int a, int &gbeg, int &len) {
        const int ul = u - u_lo;
        if (ul < kPsTabUnits) {
            gbeg = tab[(ul * 2 + a) * 2];
            len = tab[(ul * 2 + a) * 2 + 1];
        } else {
            const int trow = u + a * p.units;
            gbeg = __ldg(p.grp_ptr + trow);
            len = __ldg(p.grp_ptr + trow + 1) - gbeg;
        }
    };

    // A wait that runs out records it and turns every later wait of the CTA into a no-op, so a
    // broken pipeline ends quickly (with wrong numbers and the error word set) instead of hanging.
    auto wait_or_flag = [&](uint32_t bar, uint32_t parity, int code) {
        if (*reinterpret_cast<volatile int *>(&misc[2]) != 0) return;
        if (!ps_wait(bar, parity)) {
            *reinterpret_cast<volatile int *>(&misc[2]) = 1;
            g_linear_error = code;
        }
    };

    // ================= producer warps: one per slot, keep the ring S chunks ahead =================
    if (warp >= kPsSlots * kPsSlotWarps) {
        const int slot = warp - kPsSlots * kPsSlotWarps;
        if (lane != 0) return;
        const uint32_t full0 = smem_u32(bars + slot * 2 * S), empty0 = full0 + S * 8;
        const uint32_t stage_base = smem_u32(ps_smem + L.stages) + (uint32_t)slot * S * CG * 512u;
        const uint32_t cols_base = smem_u32(ps_smem + L.cols) + (uint32_t)slot * S * CG * 16u;
        PsChunkWalk<SWIGLU> walk;
        walk.init(p.grp_ptr, p.units, u_lo + slot, u_hi);
        for (int k = 0; walk.valid(); ++k, walk.next()) {
            const int st = k % S;
            if (k >= S) wait_or_flag(empty0 + st * 8, (uint32_t)(k / S - 1) & 1u, 3);   // chunk k - S is consumed
            int g0, ng;
            walk.get(g0, ng);
            const uint32_t bar = full0 + st * 8;
            const uint32_t cbytes = (uint32_t)ng * 512u, lbytes = (uint32_t)ng * 16u;
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(cbytes + lbytes) : "memory");
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                ::"r"(stage_base + st * (CG * 512)), "l"(p.grp_codes + (long long)g0 * 32), "r"(cbytes), "r"(bar) : "memory");
            asm volatile(
                "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                ::"r"(cols_base + st * (CG * 16)), "l"(p.grp_cols + g0), "r"(lbytes), "r"(bar) : "memory");
        }
        return;
    }

    // ================= consumer warps =================
    const int slot = warp / kPsSlotWarps, sw = warp % kPsSlotWarps;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t full0 = smem_u32(bars + slot * 2 * S), empty0 = full0 + S * 8;
    const uint32_t stage_base = smem_u32(ps_smem + L.stages) + (uint32_t)slot * S * CG * 512u;
    const uint32_t cols_base = smem_u32(ps_smem + L.cols) + (uint32_t)slot * S * CG * 16u;
    // ---- activations -> shared memory; words (2i, 2i+1) and (2i+8, 2i+9) of a tile column side by side ----
    {
        const int words = p.C * 8;
        for (int r = 0; r < vrows; ++r) {
            const uint32_t *src = p.planes + (long long)r * p.ld_w;
            uint32_t *dst = reinterpret_cast<uint32_t *>(ps_smem + L.x + r * L.x_pitch);
#pragma unroll 4
            for (int w = tid; w < words; w += kPsConsumers) {
                const int k = w & 7;
                dst[(w & ~7) + (k < 4 ? 2 * k : 2 * (k - 4) + 1)] = __ldg(src + w);
            }
        }
        asm volatile("bar.sync %0, %1;" ::"r"(kPsSlots + 1), "r"(kPsConsumers) : "memory");
    }
    const uint32_t xs_lane = smem_u32(ps_smem + L.x) + (uint32_t)min(g, vrows - 1) * (uint32_t)L.x_pitch + t * 8u;
    float *red0 = reinterpret_cast<float *>(ps_smem + L.red) + slot * 2 * kPsSlotWarps * NACC * 4 * 32;
    float(*fold_s)[16][9] = reinterpret_cast<float(*)[16][9]>(ps_smem + L.fold) + slot * 2;
    const float scale = p.round_bf16 ? round_bf16(p.scale) : p.scale;

    int c = 0;                                                  // chunks consumed by this slot so far
    int turn = 0;                                               // which warp of the slot finishes this unit
    int parity = 0;                                             // which `red` buffer this unit uses
    for (int u = u_lo + slot; u < u_hi; u += kPsSlots, turn = (turn + 1 == kPsSlotWarps) ? 0 : turn + 1, parity ^= 1) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f}, acc_gate[4] = {0.f, 0.f, 0.f, 0.f};
        int rot = sw;                                           // this warp's first group in the tile row (round robin over the slot's warps)
        for (int a = 0; a < NACC; ++a) {
            int gbeg, len;
            row_info(u, a, gbeg, len);
            (void)gbeg;
            int first = rot;                                    // this warp's first group index in the tile row
            for (int cc = 0; cc * CG < len; ++cc, ++c) {
                const int st = c % S;
                wait_or_flag(full0 + st * 8, (uint32_t)(c / S) & 1u, 2);   // on failure keeps going: every barrier is still met
                const int hi = min(len, (cc + 1) * CG);
                // once a wait has given up the stage contents are not to be trusted (column indices
                // become addresses): skip the arithmetic, keep the barrier protocol
                const bool dead = *reinterpret_cast<volatile int *>(&misc[2]) != 0;
                for (; first < hi; first += kPsSlotWarps) {
                    if (dead) continue;
                    const int gi = first - cc * CG;
                    const uint32_t codes_a = stage_base + (uint32_t)((st * CG + gi) * 512 + lane * 16);
                    const uint32_t cols_a = cols_base + (uint32_t)((st * CG + gi) * 16);
                    // only the last group of a tile row can hold padding slots
                    if (first != len - 1) ps_group<false>(acc, codes_a, cols_a, xs_lane);
                    else ps_group<true>(acc, codes_a, cols_a, xs_lane);
                }
                __syncwarp();
                if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(empty0 + st * 8) : "memory");
            }
            // keep the round robin going across the unit's tile rows
            rot = first - len;
            if (SWIGLU && a == 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) { acc_gate[i] = acc[i]; acc[i] = 0.f; }
            }
        }
        // ---- partial sums meet in shared memory; the warp whose turn it is adds them in warp order.
        // One barrier per unit: the other warps go on to the next unit, whose partial sums use
        // the other buffer; a buffer is written again only after a barrier its reader has joined.
        float *red = red0 + parity * kPsSlotWarps * NACC * 4 * 32;
        {
            float *mine = red + sw * NACC * 4 * 32;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                mine[i * 32 + lane] = SWIGLU ? acc_gate[i] : acc[i];
                if (SWIGLU) mine[(4 + i) * 32 + lane] = acc[i];
            }
        }
        ps_slot_sync(slot);
        if (sw == turn) {
#pragma unroll
            for (int i = 0; i < 4; ++i) { acc[i] = 0.f; acc_gate[i] = 0.f; }
            for (int w = 0; w < kPsSlotWarps; ++w) {
                const float *theirs = red + w * NACC * 4 * 32;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (SWIGLU) { acc_gate[i] += theirs[i * 32 + lane]; acc[i] += theirs[(4 + i) * 32 + lane]; }
                    else acc[i] += theirs[i * 32 + lane];
                }
            }
        }
        if (sw == turn) {
            // acc[0..3] = (neuron g, column 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1)
            if (p.fold > 0) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    fold_s[0][g + 8 * (i >> 1)][2 * t + (i & 1)] = SWIGLU ? acc_gate[i] : acc[i];
                    fold_s[1][g + 8 * (i >> 1)][2 * t + (i & 1)] = acc[i];
                }
                __syncwarp();
                const int rr = (int)p.real_rows;
                for (int idx = lane; idx < 16 * rr; idx += 32) {
                    const int neuron_local = idx & 15, b = idx >> 4;
                    float sa = 0.f, sb = 0.f;
                    for (int pl = 0; pl < p.fold; ++pl) {
                        sa += fold_s[0][neuron_local][pl * rr + b];
                        sb += fold_s[1][neuron_local][pl * rr + b];
                    }
                    emit_value<SWIGLU>(p, scale, u, true, b, neuron_local, sa, sb);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = 2 * t + (i & 1);
                    if (row < vrows)
                        emit_value<SWIGLU>(p, scale, u, true, row, g + 8 * (i >> 1), SWIGLU ? acc_gate[i] : acc[i], acc[i]);
                }
            }
        }
    }
}
