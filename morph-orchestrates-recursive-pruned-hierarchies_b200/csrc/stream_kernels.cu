// Streaming kernels over the 8-tile-group layout: activation-plane preparation (with the
// optional RMSNorm prologue), the block-sparse ternary linear / SwiGLU kernel used for
// decode batches and as the generic token-block path, the routing-flag kernel, and the
// fused per-MLP entry point.
//
// The linear kernel keeps the ternary tile as the A operand of mma.m16n8k16 (decoded from
// 2-bit codes straight into registers) and 8 activation rows as the B operand, so one
// fetch of a 64-byte tile serves every row of the batch.  Products are exact (+-x or 0 in
// bf16), accumulation is fp32; the per-matrix scale multiplies the finished sum, as in the
// reference combine step (morph/kernels/triton/fused_decode_step.py:1441-1459).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cstdint>
#include <mutex>
#include "common.h"
#include "decode.cuh"

namespace {

constexpr int kWarpsPerCta = 4;
constexpr int kMaxFlagCols = 4096;     // tile columns coverable by the column-activity bitmap
constexpr int kBulkStages = 2;         // shared-memory stages of the bulk-copy pipeline
constexpr int kBulkChunkGroups = 16;   // groups per stage: 8 KB of codes + 256 B of column indices
constexpr uint32_t kBulkWaitLimit = 1u << 20;   // polls of one mbarrier before the kernel gives up

// Set when a bounded mbarrier wait of the bulk-copy pipeline ran out (never in a healthy run).
__device__ int g_linear_error = 0;

struct LinearParams {
    const uint4 *grp_codes;
    const uint4 *grp_cols;
    const int *grp_ptr;
    int R, C;
    float scale;
    const uint32_t *planes;            // bf16 pairs
    long long plane_stride_w;          // in 32-bit words
    long long ld_w;                    // row stride in 32-bit words
    int n_planes;
    long long rows;
    void *out;
    int out_mode, n_out_planes;
    long long out_plane_stride, ld_out;
    int round_bf16;
    int accumulate;
    const float *gates;
    long long ld_gates;
    int cluster_size;
    int gates_on_input;
    const int *row_act;
    long long ld_row_act;
    const int *col_act;
    long long ld_col_act;
    int units;                         // output tile rows (LINEAR) or hidden tile rows (SWIGLU)
    int fold;                          // >0: the planes are folded into the 8 MMA columns (see below)
    long long real_rows;               // activation rows when fold > 0 (rows = fold * real_rows)
    const float *row_scale;            // per-output-row scales (replace `scale`) or nullptr
    // hyper-connection POST write (out_mode == MORTAR_OUT_HC): the result y feeds n carrier streams
    const float *hc_hres, *hc_hpost, *hc_in, *hc_term;
    float *hc_out;
    int hc_n;
    long long hc_ld;                   // carrier stride between tokens, in floats (n_streams * ld_out)
};

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0,
                                          uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}


__device__ __forceinline__ uint32_t smem_u32(const void *ptr) {
    return (uint32_t)__cvta_generic_to_shared(ptr);
}

__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kBulkWaitLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n.reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

__device__ __forceinline__ float round_bf16(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}

__device__ __forceinline__ void store_value(const LinearParams &p, long long row, long long col,
                                            float v) {
    if (p.out_mode == MORTAR_OUT_F32) {
        float *o = reinterpret_cast<float *>(p.out) + row * p.ld_out + col;
        *o = p.accumulate ? *o + v : v;
    } else if (p.out_mode == MORTAR_OUT_BF16) {
        __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(p.out) + row * p.ld_out + col;
        *o = __float2bfloat16_rn(p.accumulate ? __bfloat162float(*o) + v : v);
    } else if (p.out_mode == MORTAR_OUT_HC) {
        // out[i][col] = sum_j Hres[i][j] * h[j][col] + Hpost_row[i] * y[col] (+ term[col]) for the n
        // streams of this token (fused_hyper_connection.py:933-977); every h[j][col] is read before
        // the first write, so the carrier may be updated in place
        const int n = p.hc_n;
        const float *hres = p.hc_hres + row * n * n, *hpost = p.hc_hpost + row * n;
        const float *hin = p.hc_in + row * p.hc_ld + col;
        float *o = p.hc_out + row * p.hc_ld + col;
        const float term = p.hc_term != nullptr ? p.hc_term[row * p.ld_out + col] : 0.f;
        float hj[8];
        for (int j = 0; j < n; ++j) hj[j] = hin[j * p.ld_out];
        for (int i = 0; i < n; ++i) {
            float acc = 0.f;
            for (int j = 0; j < n; ++j) acc += hres[i * n + j] * hj[j];
            acc += hpost[i] * v;
            if (p.hc_term != nullptr) acc += term;
            o[i * p.ld_out] = acc;
        }
    } else {
        __nv_bfloat16 *o = reinterpret_cast<__nv_bfloat16 *>(p.out) + row * p.ld_out + col;
        float r = v;
        for (int pl = 0; pl < p.n_out_planes; ++pl) {
            __nv_bfloat16 h = __float2bfloat16_rn(r);
            o[pl * p.out_plane_stride] = h;
            r -= __bfloat162float(h);
        }
    }
}

// Finished sums of one output element -> scale, SwiGLU and cluster gate (with the reference's
// bf16 rounding points when asked for), then the store.  sum_a is the gate (or only) tile row's
// sum, sum_b the up tile row's.
template <bool SWIGLU>
__device__ __forceinline__ void emit_value(const LinearParams &p, float scale, int unit, bool active,
                                           long long row, int neuron_local, float sum_a, float sum_b) {
    const int neuron = unit * 16 + neuron_local;
    float v;
    if (SWIGLU) {
        float gv = scale * sum_a;
        float uv = scale * sum_b;
        float gate = 1.f;
        if (p.gates != nullptr) gate = p.gates[row * p.ld_gates + neuron / p.cluster_size];
        if (p.round_bf16) {
            gv = round_bf16(gv);
            uv = round_bf16(uv);
            const float sg = round_bf16(gv / (1.f + expf(-gv)));
            v = round_bf16(sg * uv);
            if (p.gates != nullptr) v = round_bf16(v * round_bf16(gate));
        } else {
            v = gv * (1.f / (1.f + expf(-gv))) * uv;
            if (p.gates != nullptr) v *= gate;
        }
        if (!active || (p.gates != nullptr && !(gate > 0.f))) v = 0.f;
    } else {
        v = (p.row_scale != nullptr ? p.row_scale[neuron] : scale) * sum_a;
        if (!active) v = 0.f;
    }
    store_value(p, row, neuron, v);
}

// One 8-tile group against NT blocks of 8 activation rows and P planes.  Activation fragments
// of SB slots are fetched together before any of them is consumed, so the loads overlap
// instead of each waiting behind the previous MMA.  CHECK = false is the all-slots-live case.
// SCOLS: the eight column indices are read one by one from shared memory (address `cols_s`,
// load/store pipe) instead of being extracted from the register quad `cl` (integer pipe).
template <int NT, int P, int SB, bool CHECK, bool SCOLS = false>
__device__ __forceinline__ void group_mma(float (&acc)[NT][4], const uint4 cw, const uint4 cl,
                                          const uint32_t *const (&xb)[NT], long long plane_stride_w,
                                          const uint32_t *col_active, uint32_t cols_s = 0) {
    const uint32_t cws[4] = {cw.x, cw.y, cw.z, cw.w};
    const uint32_t cls[4] = {cl.x, cl.y, cl.z, cl.w};
#pragma unroll
    for (int s0 = 0; s0 < 8; s0 += SB) {
        uint32_t bf[SB][NT][P][2];
        bool live[SB];
#pragma unroll
        for (int ss = 0; ss < SB; ++ss) {
            const int s = s0 + ss;
            uint32_t col;
            if (SCOLS) asm volatile("ld.shared.u16 %0, [%1];" : "=r"(col) : "r"(cols_s + 2u * s));
            else col = (s & 1) ? (cls[s >> 1] >> 16) : (cls[s >> 1] & 0xffffu);
            live[ss] = true;
            if (CHECK) {
                live[ss] = (col != 0xffffu);                 // padding slots end a row
                if (col_active != nullptr && live[ss]) live[ss] = ((col_active[col >> 5] >> (col & 31u)) & 1u) != 0;
            }
            if (live[ss]) {
#pragma unroll
                for (int n = 0; n < NT; ++n) {
                    const uint32_t *px = xb[n] + (long long)col * 8;
#pragma unroll
                    for (int pl = 0; pl < P; ++pl) {
                        bf[ss][n][pl][0] = __ldg(px);
                        bf[ss][n][pl][1] = __ldg(px + 4);
                        px += plane_stride_w;
                    }
                }
            }
        }
#pragma unroll
        for (int ss = 0; ss < SB; ++ss) {
            const int s = s0 + ss;
            if (live[ss]) {
                const uint32_t word = cws[s >> 1];
                uint32_t af[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) af[i] = mortar_decode_pair(word, (s & 1) * 4 + i);
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int pl = 0; pl < P; ++pl)
                        mma_16816(acc[n], af, bf[ss][n][pl][0], bf[ss][n][pl][1]);
            }
        }
    }
}

// One CTA = 4 warps; WPR warps cooperate on one unit (a tile row, or for SWIGLU a hidden
// tile row = gate row u and up row u+units), 4/WPR units per CTA.  blockIdx.y selects a
// block of 8*NT activation rows.
//
// BULK (needs WPR = 4, one unit per CTA): the unit's groups are not read with per-lane loads but
// staged into shared memory by bulk asynchronous copies (one elected thread, mbarrier
// completion), kBulkStages chunks of kBulkChunkGroups groups in flight per CTA from the first
// instruction on.  That is what keeps enough bytes in flight to stream a matrix much larger
// than L2; the group-to-warp assignment and the summation order are those of the plain path,
// so both give bit-identical results.
template <int NT, int P, bool SWIGLU, int WPR, bool BULK>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 1)
bcsr_stream_kernel(const LinearParams p) {
    static_assert(!BULK || WPR == kWarpsPerCta, "the bulk pipeline serves one unit per CTA");
    constexpr int UPC = kWarpsPerCta / WPR;
    // tile slots whose activation fragments are fetched together before any of them is
    // consumed, so the loads overlap instead of each waiting behind the previous MMA
    constexpr int SB = (16 / (NT * P) >= 8) ? 8 : (16 / (NT * P) >= 4) ? 4 : (16 / (NT * P) >= 2) ? 2 : 1;
    constexpr int NACC = SWIGLU ? 2 : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int unit_local = warp / WPR, sub = warp % WPR;
    const int unit = blockIdx.x * UPC + unit_local;
    const long long row0 = (long long)blockIdx.y * (8 * NT);
    // with folded planes the MMA columns are virtual rows; gates and flags are per real row
    const int nrows = p.fold > 0 ? (int)p.real_rows : (int)min((long long)(8 * NT), p.rows - row0);

    constexpr int kRedFloats = (WPR > 1) ? UPC * (WPR - 1) * NACC * NT * 4 * 32 : 1;
    constexpr int kStageBytes = BULK ? kBulkStages * kBulkChunkGroups * 512 : 0;
    // the cross-warp sum reuses the stage memory once every chunk has been consumed
    constexpr int kPoolBytes = kStageBytes > kRedFloats * 4 ? kStageBytes : kRedFloats * 4;
    __shared__ __align__(128) unsigned char pool[kPoolBytes];
    __shared__ __align__(16) uint4 cols_s[BULK ? kBulkStages * kBulkChunkGroups : 1];
    __shared__ __align__(8) unsigned long long bars[BULK ? 2 * kBulkStages : 1];   // full[], empty[]
    float *red = reinterpret_cast<float *>(pool);
    __shared__ uint32_t col_active[kMaxFlagCols / 32];       // one bit per tile column
    if (BULK && threadIdx.x == 0) {
        for (int i = 0; i < kBulkStages; ++i) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&bars[i])));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(&bars[kBulkStages + i])),
                         "r"(kWarpsPerCta));
        }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (BULK) __syncthreads();

    // Column-activity bitmap for this block of rows (only built for small batches).
    const bool use_cact = (p.col_act != nullptr) || (p.gates_on_input != 0);
    if (use_cact) {
        for (int wd = threadIdx.x; wd < (p.C + 31) / 32; wd += blockDim.x) {
            uint32_t bits = 0;
            for (int j = 0; j < 32 && wd * 32 + j < p.C; ++j) {
                const int c = wd * 32 + j;
                int any = 0;
                if (p.col_act != nullptr) {
                    for (int b = 0; b < nrows; ++b) any |= p.col_act[(row0 + b) * p.ld_col_act + c];
                } else {
                    const int lo = (c * 16) / p.cluster_size, hi = (c * 16 + 15) / p.cluster_size;
                    for (int b = 0; b < nrows; ++b)
                        for (int k = lo; k <= hi; ++k)
                            any |= (p.gates[(row0 + b) * p.ld_gates + k] > 0.f);
                }
                bits |= (uint32_t)(any != 0) << j;
            }
            col_active[wd] = bits;
        }
        __syncthreads();
    }

    const bool unit_valid = unit < p.units;
    bool active = unit_valid;
    if (unit_valid && (p.row_act != nullptr || (SWIGLU && p.gates != nullptr))) {
        int any = 0;
        for (int b = lane; b < nrows; b += 32) {
            if (p.row_act != nullptr) {
                any |= p.row_act[(row0 + b) * p.ld_row_act + unit];
            } else {
                const int lo = (unit * 16) / p.cluster_size, hi = (unit * 16 + 15) / p.cluster_size;
                for (int k = lo; k <= hi; ++k) any |= (p.gates[(row0 + b) * p.ld_gates + k] > 0.f);
            }
        }
        active = __any_sync(0xffffffffu, any != 0);
    }

    float acc[NACC][NT][4];
#pragma unroll
    for (int a = 0; a < NACC; ++a)
#pragma unroll
        for (int n = 0; n < NT; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[a][n][i] = 0.f;

    if (active) {
        const uint32_t *xb[NT];
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            long long tok = row0 + n * 8 + g;
            if (tok > p.rows - 1) tok = p.rows - 1;      // clamped rows compute discarded values
            xb[n] = p.planes + tok * p.ld_w + t;
        }
        if constexpr (BULK) {
            constexpr int S = kBulkStages, CG = kBulkChunkGroups;
            const uint4 *codes_s = reinterpret_cast<const uint4 *>(pool);
            int gb[NACC], nch[NACC], len[NACC], total = 0;
#pragma unroll
            for (int a = 0; a < NACC; ++a) {
                const int trow = unit + a * p.units;
                gb[a] = p.grp_ptr[trow];
                len[a] = p.grp_ptr[trow + 1] - gb[a];
                nch[a] = (len[a] + CG - 1) / CG;
                total += nch[a];
            }
            // chunk c of the unit -> its first group and group count
            auto chunk_of = [&](int c, int &g0, int &ng) {
                int a = 0;
                if (NACC > 1 && c >= nch[0]) { a = NACC - 1; c -= nch[0]; }
                g0 = gb[a] + c * CG;
                ng = min(CG, len[a] - c * CG);
            };
            auto issue = [&](int c) {
                int g0, ng;
                chunk_of(c, g0, ng);
                const int st = c % S;
                const uint32_t bar = smem_u32(&bars[st]);
                const uint32_t cbytes = (uint32_t)ng * 512u, lbytes = (uint32_t)ng * 16u;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar),
                             "r"(cbytes + lbytes) : "memory");
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                    ::"r"(smem_u32(pool + st * (CG * 512))), "l"(p.grp_codes + (long long)g0 * 32), "r"(cbytes),
                    "r"(bar) : "memory");
                asm volatile(
                    "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                    ::"r"(smem_u32(cols_s + st * CG)), "l"(p.grp_cols + g0), "r"(lbytes), "r"(bar) : "memory");
            };
            if (threadIdx.x == 0)
                for (int c = 0; c < total && c < S; ++c) issue(c);
            int c = 0, done = 0;
            bool ok = true;
#pragma unroll
            for (int a = 0; a < NACC; ++a) {
                for (int cc = 0; cc < nch[a] && ok; ++cc, ++c) {
                    const int st = c % S;
                    const uint32_t ph = (uint32_t)(c / S) & 1u;
                    const int ng = min(CG, len[a] - cc * CG);
                    ok = mbar_wait_bounded(smem_u32(&bars[st]), ph);
                    if (!ok) { g_linear_error = 1; break; }
                    for (int gi = ((sub - done) % WPR + WPR) % WPR; gi < ng; gi += WPR) {
                        const uint4 cw = codes_s[(st * CG + gi) * 32 + lane];
                        const uint4 cl = make_uint4(0, 0, 0, 0);
                        const uint32_t cols_a = smem_u32(cols_s + st * CG + gi);
                        // only the last group of a tile row can hold padding slots
                        if (!use_cact && cc * CG + gi != len[a] - 1)
                            group_mma<NT, P, SB, false, true>(acc[a], cw, cl, xb, p.plane_stride_w, nullptr, cols_a);
                        else
                            group_mma<NT, P, SB, true, true>(acc[a], cw, cl, xb, p.plane_stride_w,
                                                             use_cact ? col_active : nullptr, cols_a);
                    }
                    if (c + S < total) {
                        // hand the stage back; the elected thread refills it once all four warps have
                        __syncwarp();
                        if (lane == 0)
                            asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(&bars[S + st])) : "memory");
                        if (threadIdx.x == 0) {
                            if (mbar_wait_bounded(smem_u32(&bars[S + st]), ph)) issue(c + S);
                            else g_linear_error = 1;
                        }
                        __syncwarp();
                    }
                }
                done += len[a];
            }
        } else {
        int done = 0;   // groups of earlier tile rows of this unit, keeps the round-robin going
#pragma unroll
        for (int a = 0; a < NACC; ++a) {
            const int trow = unit + a * p.units;
            const int gbeg = p.grp_ptr[trow], gend = p.grp_ptr[trow + 1];
            int grp = gbeg + ((sub - done) % WPR + WPR) % WPR;
            uint4 cw = make_uint4(0, 0, 0, 0), cl = make_uint4(0, 0, 0, 0);
            if (grp < gend) {
                cw = __ldg(p.grp_codes + (long long)grp * 32 + lane);
                cl = __ldg(p.grp_cols + grp);
            }
            while (grp < gend) {
                const int ngrp = grp + WPR;
                uint4 ncw = cw, ncl = cl;
                if (ngrp < gend) {
                    ncw = __ldg(p.grp_codes + (long long)ngrp * 32 + lane);
                    ncl = __ldg(p.grp_cols + ngrp);
                }
                // a group whose last slot is a real tile has no padding: skip the per-slot tests
                if (!use_cact && (cl.w >> 16) != 0xffffu)
                    group_mma<NT, P, SB, false>(acc[a], cw, cl, xb, p.plane_stride_w, col_active);
                else
                    group_mma<NT, P, SB, true>(acc[a], cw, cl, xb, p.plane_stride_w,
                                               use_cact ? col_active : nullptr);
                cw = ncw; cl = ncl; grp = ngrp;
            }
            done += gend - gbeg;
        }
        }
    }

    if (WPR > 1) {
        // fixed-order cross-warp sum: warps sub=1..WPR-1 publish, warp sub=0 adds in order
        float *mine = red + ((unit_local * (WPR - 1) + (sub > 0 ? sub - 1 : 0)) * NACC * NT * 4) * 32;
        if (BULK) __syncthreads();      // every warp is done reading the stages that `red` reuses
        if (sub > 0) {
#pragma unroll
            for (int a = 0; a < NACC; ++a)
#pragma unroll
                for (int n = 0; n < NT; ++n)
#pragma unroll
                    for (int i = 0; i < 4; ++i) mine[((a * NT + n) * 4 + i) * 32 + lane] = acc[a][n][i];
        }
        __syncthreads();
        if (sub == 0) {
            for (int w = 0; w < WPR - 1; ++w) {
                const float *theirs = red + ((unit_local * (WPR - 1) + w) * NACC * NT * 4) * 32;
#pragma unroll
                for (int a = 0; a < NACC; ++a)
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            acc[a][n][i] += theirs[((a * NT + n) * 4 + i) * 32 + lane];
            }
        }
    }
    if (sub != 0 || !unit_valid) return;

    // Epilogue.  acc[.][n][0..3] = (neuron g, row 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1).
    const float scale = p.round_bf16 ? round_bf16(p.scale) : p.scale;
    auto emit = [&](long long row, int neuron_local, float sum_a, float sum_b) {
        emit_value<SWIGLU>(p, scale, unit, active, row, neuron_local, sum_a, sum_b);
    };
    if (NT == 1 && P == 1 && p.fold > 0) {
        // Folded planes: MMA column pl*real_rows + b holds plane pl of activation row b, so the
        // value of row b is the sum of `fold` columns.  Stage the 16x8 tile and combine.
        __shared__ float fold_s[UPC][NACC][16][9];
#pragma unroll
        for (int a = 0; a < NACC; ++a)
#pragma unroll
            for (int i = 0; i < 4; ++i) fold_s[unit_local][a][g + 8 * (i >> 1)][2 * t + (i & 1)] = acc[a][0][i];
        __syncwarp();
        const int rr = (int)p.real_rows;
        for (int idx = lane; idx < 16 * rr; idx += 32) {
            const int neuron_local = idx & 15, b = idx >> 4;
            float sa = 0.f, sb = 0.f;
            for (int pl = 0; pl < p.fold; ++pl) {
                sa += fold_s[unit_local][0][neuron_local][pl * rr + b];
                sb += fold_s[unit_local][NACC - 1][neuron_local][pl * rr + b];
            }
            emit(b, neuron_local, sa, sb);
        }
        return;
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const long long row = row0 + n * 8 + 2 * t + (i & 1);
            if (row >= p.rows) continue;
            emit(row, g + 8 * (i >> 1), acc[0][n][i], acc[NACC - 1][n][i]);
        }
    }
}


// ---- ReMoE per-token tile gather -----------------------------------------------------------
// For batches of more than 8 rows the any-row-active test of the kernel above almost never
// skips a hidden tile row (each row activates its own quarter of the groups).  Here the rows are
// regrouped per hidden tile row instead: route_gather_kernel lists, for every hidden tile row,
// the rows whose gate over it is positive (ascending), and bcsr_gather_kernel runs the gate and
// up tile rows of a unit over blocks of 8*NT LISTED rows only -- the per-stream skip of the
// reference's decode kernel (fused_decode_step.py:1371-1390) with the weights still fetched once
// per block of rows instead of once per row.  Rows that are not listed keep the zeros the caller
// put into the output, which is what the multiply by a zero gate gives (transformer.py:419-427).

// gates[rows, n_clusters] -> cnt[units], list[units][ld_list]: one warp per hidden tile row.
__global__ void __launch_bounds__(128)
route_gather_kernel(const float *gates, long long ld_gates, int rows, int cluster_size, int units,
                    int *cnt, int *list, long long ld_list) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int u = blockIdx.x * 4 + warp;
    if (u >= units) return;
    const int lo = (u * 16) / cluster_size, hi = (u * 16 + 15) / cluster_size;
    int base = 0;
    for (int t0 = 0; t0 < rows; t0 += 32) {
        const int t = t0 + lane;
        bool act = false;
        if (t < rows)
            for (int k = lo; k <= hi; ++k) act |= gates[(long long)t * ld_gates + k] > 0.f;
        const uint32_t m = __ballot_sync(0xffffffffu, act);
        if (act) list[(long long)u * ld_list + base + __popc(m & ((1u << lane) - 1u))] = t;
        base += __popc(m);
    }
    if (lane == 0) cnt[u] = base;
}

template <int NT, int P, int WPR>
__global__ void __launch_bounds__(kWarpsPerCta * 32, 1)
bcsr_gather_kernel(const LinearParams p, const int *__restrict__ cnt, const int *__restrict__ list,
                   long long ld_list) {
    constexpr int UPC = kWarpsPerCta / WPR;
    constexpr int SB = (16 / (NT * P) >= 8) ? 8 : (16 / (NT * P) >= 4) ? 4 : (16 / (NT * P) >= 2) ? 2 : 1;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int unit_local = warp / WPR, sub = warp % WPR;
    const int unit = blockIdx.x * UPC + unit_local;
    const bool unit_valid = unit < p.units;
    const int my_cnt = unit_valid ? cnt[unit] : 0;
    const int *my_list = list + (long long)(unit_valid ? unit : 0) * ld_list;

    constexpr int kRedFloats = (WPR > 1) ? UPC * (WPR - 1) * 2 * NT * 4 * 32 : 1;
    __shared__ __align__(16) float red[kRedFloats];
    __shared__ int cnt_s[UPC];
    if (sub == 0 && lane == 0) cnt_s[unit_local] = my_cnt;
    __syncthreads();
    int max_cnt = 0;                        // the warps of a CTA iterate together (shared-memory sum)
#pragma unroll
    for (int k = 0; k < UPC; ++k) max_cnt = max(max_cnt, cnt_s[k]);
    const float scale = p.round_bf16 ? round_bf16(p.scale) : p.scale;

    for (int j = blockIdx.y; j * (8 * NT) < max_cnt; j += gridDim.y) {
        const int base = j * (8 * NT);
        const bool live = base < my_cnt;
        float acc[2][NT][4];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int n = 0; n < NT; ++n)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[a][n][i] = 0.f;
        if (live) {
            const uint32_t *xb[NT];
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                const int idx = min(base + n * 8 + g, my_cnt - 1);      // past the end: discarded values
                xb[n] = p.planes + (long long)__ldg(my_list + idx) * p.ld_w + t;
            }
            int done = 0;
#pragma unroll
            for (int a = 0; a < 2; ++a) {
                const int trow = unit + a * p.units;
                const int gbeg = p.grp_ptr[trow], gend = p.grp_ptr[trow + 1];
                int grp = gbeg + ((sub - done) % WPR + WPR) % WPR;
                uint4 cw = make_uint4(0, 0, 0, 0), cl = make_uint4(0, 0, 0, 0);
                if (grp < gend) {
                    cw = __ldg(p.grp_codes + (long long)grp * 32 + lane);
                    cl = __ldg(p.grp_cols + grp);
                }
                while (grp < gend) {
                    const int ngrp = grp + WPR;
                    uint4 ncw = cw, ncl = cl;
                    if (ngrp < gend) {
                        ncw = __ldg(p.grp_codes + (long long)ngrp * 32 + lane);
                        ncl = __ldg(p.grp_cols + ngrp);
                    }
                    if ((cl.w >> 16) != 0xffffu) group_mma<NT, P, SB, false>(acc[a], cw, cl, xb, p.plane_stride_w, nullptr);
                    else group_mma<NT, P, SB, true>(acc[a], cw, cl, xb, p.plane_stride_w, nullptr);
                    cw = ncw; cl = ncl; grp = ngrp;
                }
                done += gend - gbeg;
            }
        }
        if (WPR > 1) {
            float *mine = red + ((unit_local * (WPR - 1) + (sub > 0 ? sub - 1 : 0)) * 2 * NT * 4) * 32;
            if (sub > 0) {
#pragma unroll
                for (int a = 0; a < 2; ++a)
#pragma unroll
                    for (int n = 0; n < NT; ++n)
#pragma unroll
                        for (int i = 0; i < 4; ++i) mine[((a * NT + n) * 4 + i) * 32 + lane] = acc[a][n][i];
            }
            __syncthreads();
            if (sub == 0) {
                for (int w = 0; w < WPR - 1; ++w) {
                    const float *theirs = red + ((unit_local * (WPR - 1) + w) * 2 * NT * 4) * 32;
#pragma unroll
                    for (int a = 0; a < 2; ++a)
#pragma unroll
                        for (int n = 0; n < NT; ++n)
#pragma unroll
                            for (int i = 0; i < 4; ++i) acc[a][n][i] += theirs[((a * NT + n) * 4 + i) * 32 + lane];
                }
            }
            __syncthreads();                    // `red` is free again for the next block of rows
        }
        if (sub == 0 && live) {
            // acc[.][n][0..3] = (neuron g, column 2t), (g, 2t+1), (g+8, 2t), (g+8, 2t+1) of block n
#pragma unroll
            for (int n = 0; n < NT; ++n) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int idx = base + n * 8 + 2 * t + (i & 1);
                    if (idx >= my_cnt) continue;
                    emit_value<true>(p, scale, unit, true, __ldg(my_list + idx), g + 8 * (i >> 1), acc[0][n][i],
                                     acc[1][n][i]);
                }
            }
        }
    }
}

#include "gemv_persistent.cuh"

// x[rows, cols] -> bf16 planes, optional RMSNorm prologue.  One CTA per row.
template <typename T>
__global__ void __launch_bounds__(256)
act_prep_kernel(const T *x, long long ldx, int cols, const float *rms_w, float eps,
                __nv_bfloat16 *planes, int n_planes, long long plane_stride, long long ld_planes) {
    const long long row = blockIdx.x;
    const T *xr = x + row * ldx;
    float inv = 1.f;
    if (rms_w != nullptr) {
        float ss = 0.f;
        for (int c = threadIdx.x; c < cols; c += blockDim.x) {
            const float v = (float)xr[c];
            ss += v * v;
        }
        __shared__ float part[8];
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
        for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += part[w];
        inv = 1.f / sqrtf(tot / (float)cols + eps);
    }
    for (int c = threadIdx.x; c < cols; c += blockDim.x) {
        float v = (float)xr[c];
        if (rms_w != nullptr) v = (v * inv) * rms_w[c];
        __nv_bfloat16 *o = planes + row * ld_planes + c;
        for (int pl = 0; pl < n_planes; ++pl) {
            const __nv_bfloat16 h = __float2bfloat16_rn(v);
            o[pl * plane_stride] = h;
            v -= __bfloat162float(h);
        }
    }
}

__global__ void route_flags_kernel(const float *gates, long long ld_gates, const int *rlo,
                                   const int *rhi, int n_row, const int *clo, const int *chi,
                                   int n_col, int *ract, long long ld_ract, int *cact,
                                   long long ld_cact) {
    const long long b = blockIdx.x;
    const float *gb = gates + b * ld_gates;
    for (int i = threadIdx.x; i < n_row; i += blockDim.x)
        ract[b * ld_ract + i] = (gb[rlo[i]] > 0.f) | (gb[rhi[i]] > 0.f);
    for (int i = threadIdx.x; i < n_col; i += blockDim.x)
        cact[b * ld_cact + i] = (gb[clo[i]] > 0.f) | (gb[chi[i]] > 0.f);
}

template <int NT, int P, bool SWIGLU>
int launch_wpr(const LinearParams &p, int wpr, bool bulk, unsigned grid_y, cudaStream_t st) {
    const int upc = kWarpsPerCta / wpr;
    dim3 grid((p.units + upc - 1) / upc, grid_y);
    if (wpr == 4 && bulk) bcsr_stream_kernel<NT, P, SWIGLU, 4, true><<<grid, kWarpsPerCta * 32, 0, st>>>(p);
    else if (wpr == 4) bcsr_stream_kernel<NT, P, SWIGLU, 4, false><<<grid, kWarpsPerCta * 32, 0, st>>>(p);
    else if (wpr == 2) bcsr_stream_kernel<NT, P, SWIGLU, 2, false><<<grid, kWarpsPerCta * 32, 0, st>>>(p);
    else bcsr_stream_kernel<NT, P, SWIGLU, 1, false><<<grid, kWarpsPerCta * 32, 0, st>>>(p);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

template <int P, bool SWIGLU>
int launch_nt(const LinearParams &p, int wpr, bool bulk, cudaStream_t st) {
    // Small matrices and small batches are latency-bound: prefer many light CTAs (8 rows each,
    // weights re-read from L2 per row block) until the grid covers the GPU a few times over.
    const int upc = kWarpsPerCta / wpr;
    const long long ctas_x = (p.units + upc - 1) / upc;
    const long long blocks8 = (p.rows + 7) / 8;
    if (p.rows <= 8 || ctas_x * blocks8 <= 148 * 16) {
        if (blocks8 > 65535) return MORTAR_ERR_CAPACITY;
        return launch_wpr<1, P, SWIGLU>(p, wpr, bulk, (unsigned)blocks8, st);
    }
    const long long blocks16 = (p.rows + 15) / 16;
    if (p.rows <= 16 || ctas_x * blocks16 <= 148 * 16) {
        if (blocks16 > 65535) return MORTAR_ERR_CAPACITY;
        return launch_wpr<2, P, SWIGLU>(p, wpr, bulk, (unsigned)blocks16, st);
    }
    const long long blocks = (p.rows + 31) / 32;
    if (blocks > 65535) return MORTAR_ERR_CAPACITY;
    return launch_wpr<4, P, SWIGLU>(p, wpr, bulk, (unsigned)blocks, st);
}

template <bool SWIGLU>
int launch_planes(const LinearParams &p, int wpr, bool bulk, cudaStream_t st) {
    if (p.n_planes == 1) return launch_nt<1, SWIGLU>(p, wpr, bulk, st);
    if (p.n_planes == 2) return launch_nt<2, SWIGLU>(p, wpr, bulk, st);
    return launch_nt<3, SWIGLU>(p, wpr, bulk, st);
}


template <int NT, int P>
int launch_gather_wpr(const LinearParams &p, int wpr, const int *cnt, const int *list, long long ld_list,
                      cudaStream_t st) {
    const int upc = kWarpsPerCta / wpr;
    const long long ctas_x = (p.units + upc - 1) / upc;
    long long blocks = (p.rows + 8 * NT - 1) / (8 * NT);
    // enough CTAs per unit to cover the GPU a few times; each CTA loops over its unit's blocks
    const long long cap = (148 * 24 + ctas_x - 1) / ctas_x;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    dim3 grid((unsigned)ctas_x, (unsigned)blocks);
    if (wpr == 4) bcsr_gather_kernel<NT, P, 4><<<grid, kWarpsPerCta * 32, 0, st>>>(p, cnt, list, ld_list);
    else if (wpr == 2) bcsr_gather_kernel<NT, P, 2><<<grid, kWarpsPerCta * 32, 0, st>>>(p, cnt, list, ld_list);
    else bcsr_gather_kernel<NT, P, 1><<<grid, kWarpsPerCta * 32, 0, st>>>(p, cnt, list, ld_list);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

template <int P>
int launch_gather(const LinearParams &p, int wpr, const int *cnt, const int *list, long long ld_list,
                  cudaStream_t st) {
    // a unit sees about a quarter of the rows: pick the rows-per-CTA step for that count
    if (p.rows <= 128) return launch_gather_wpr<1, P>(p, wpr, cnt, list, ld_list, st);
    if (p.rows <= 512) return launch_gather_wpr<2, P>(p, wpr, cnt, list, ld_list, st);
    return launch_gather_wpr<4, P>(p, wpr, cnt, list, ld_list, st);
}

template <bool SWIGLU>
int launch_persistent(const LinearParams &p, cudaStream_t st) {
    const PsLayout L = ps_layout(p.C, (int)p.rows, SWIGLU);
    int dev = 0, sms = 0;
    MORTAR_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MORTAR_ERR_CAPACITY;
    {
        // once per device: SM count and the opt-in to the full shared-memory carve-out
        static std::mutex mu;
        static int sm_count[64] = {0};
        std::lock_guard<std::mutex> lock(mu);
        if (sm_count[dev] == 0) {
            int v = 0;
            MORTAR_CUDA_CHECK(cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev));
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(gemv_persistent_kernel<SWIGLU>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, kPsMaxSmem));
            sm_count[dev] = v;
        }
        sms = sm_count[dev];
    }
    const int grid = p.units < sms ? p.units : sms;
    gemv_persistent_kernel<SWIGLU><<<grid, kPsWarps * 32, L.total, st>>>(p);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

inline bool aligned(const void *ptr, size_t a) { return (reinterpret_cast<uintptr_t>(ptr) % a) == 0; }

}  // namespace

extern "C" int mortar_act_prep(const void *x, int x_dtype, int64_t rows, int32_t cols, int64_t ldx,
                               const float *rms_weight, float eps, void *planes, int32_t n_planes,
                               int64_t plane_stride, int64_t ld_planes, void *stream) {
    if (!x || !planes) return MORTAR_ERR_NULL;
    if (rows < 0 || cols <= 0 || ldx < cols || ld_planes < cols) return MORTAR_ERR_SHAPE;
    if (n_planes < 1 || n_planes > 3) return MORTAR_ERR_DTYPE;
    if (rows == 0) return MORTAR_OK;
    if (rows > 0x7fffffffLL) return MORTAR_ERR_CAPACITY;
    cudaStream_t st = (cudaStream_t)stream;
    __nv_bfloat16 *pl = reinterpret_cast<__nv_bfloat16 *>(planes);
    if (x_dtype == MORTAR_F32)
        act_prep_kernel<float><<<(unsigned)rows, 256, 0, st>>>(
            reinterpret_cast<const float *>(x), ldx, cols, rms_weight, eps, pl, n_planes,
            plane_stride, ld_planes);
    else if (x_dtype == MORTAR_BF16)
        act_prep_kernel<__nv_bfloat16><<<(unsigned)rows, 256, 0, st>>>(
            reinterpret_cast<const __nv_bfloat16 *>(x), ldx, cols, rms_weight, eps, pl, n_planes,
            plane_stride, ld_planes);
    else
        return MORTAR_ERR_DTYPE;
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

static int linear_impl(const mortar_stream *w, const void *planes, int32_t n_planes,
                       int64_t plane_stride, int64_t ld_planes, int64_t rows, void *out,
                       int32_t out_mode, int32_t n_out_planes, int64_t out_plane_stride,
                       int64_t ld_out, int32_t flags, const float *gates, int64_t ld_gates,
                       int32_t cluster_size, const int32_t *row_act, int64_t ld_row_act,
                       const int32_t *col_act, int64_t ld_col_act, const mortar_hc_post *hc, void *stream) {
    if (hc != nullptr) {
        if (!hc->hres || !hc->hpost_row || !hc->carrier_in || !hc->carrier_out) return MORTAR_ERR_NULL;
        if (hc->n_streams < 1 || hc->n_streams > 8) return MORTAR_ERR_SHAPE;
        if (flags & (MORTAR_FLAG_SWIGLU | MORTAR_FLAG_ACCUMULATE)) return MORTAR_ERR_UNSUPPORTED;
        out = hc->carrier_out;
        out_mode = MORTAR_OUT_HC;
    } else if (out_mode == MORTAR_OUT_HC) {
        return MORTAR_ERR_DTYPE;
    }
    if (!w || !planes || !out || !w->grp_ptr) return MORTAR_ERR_NULL;
    if (w->n_groups > 0 && (!w->grp_codes || !w->grp_cols)) return MORTAR_ERR_NULL;
    if (w->tile_rows <= 0 || w->tile_cols <= 0 || w->tile_cols > 65534 || rows < 0)
        return MORTAR_ERR_SHAPE;
    if (n_planes < 1 || n_planes > 3) return MORTAR_ERR_DTYPE;
    if (out_mode < MORTAR_OUT_F32 || out_mode > MORTAR_OUT_HC) return MORTAR_ERR_DTYPE;
    if (out_mode == MORTAR_OUT_PLANES && (n_out_planes < 1 || n_out_planes > 3)) return MORTAR_ERR_DTYPE;
    const bool swiglu = (flags & MORTAR_FLAG_SWIGLU) != 0;
    if (swiglu && (w->tile_rows % 2)) return MORTAR_ERR_SHAPE;
    if (swiglu && w->row_scale) return MORTAR_ERR_UNSUPPORTED;
    const int units = swiglu ? w->tile_rows / 2 : w->tile_rows;
    if (ld_planes < (int64_t)w->tile_cols * 16 || ld_out < (int64_t)units * 16) return MORTAR_ERR_SHAPE;
    if (!aligned(planes, 4) || (ld_planes & 1) || (plane_stride & 1)) return MORTAR_ERR_ALIGN;
    if (!aligned(w->grp_codes, 16) || !aligned(w->grp_cols, 16)) return MORTAR_ERR_ALIGN;
    const bool gates_on_input = (flags & MORTAR_FLAG_GATES_ON_INPUT) != 0;
    if (gates && cluster_size <= 0) return MORTAR_ERR_SHAPE;
    if (gates && !swiglu && !gates_on_input) return MORTAR_ERR_UNSUPPORTED;
    if (rows == 0) return MORTAR_OK;

    LinearParams p;
    p.grp_codes = reinterpret_cast<const uint4 *>(w->grp_codes);
    p.grp_cols = reinterpret_cast<const uint4 *>(w->grp_cols);
    p.grp_ptr = w->grp_ptr;
    p.R = w->tile_rows; p.C = w->tile_cols; p.scale = w->scale;
    p.planes = reinterpret_cast<const uint32_t *>(planes);
    p.plane_stride_w = plane_stride / 2; p.ld_w = ld_planes / 2; p.n_planes = n_planes;
    p.rows = rows;
    p.out = out; p.out_mode = out_mode; p.n_out_planes = n_out_planes;
    p.out_plane_stride = out_plane_stride; p.ld_out = ld_out;
    p.round_bf16 = (flags & MORTAR_FLAG_ROUND_BF16) != 0;
    p.accumulate = (flags & MORTAR_FLAG_ACCUMULATE) != 0;
    if (p.accumulate && out_mode == MORTAR_OUT_PLANES) return MORTAR_ERR_UNSUPPORTED;
    p.gates = gates; p.ld_gates = ld_gates; p.cluster_size = cluster_size > 0 ? cluster_size : 1;
    // activity bitmaps over input columns are only worth building for small batches
    const bool small = rows <= 8 && w->tile_cols <= kMaxFlagCols;
    p.gates_on_input = (gates_on_input && gates && small) ? 1 : 0;
    p.row_act = row_act; p.ld_row_act = ld_row_act;
    p.col_act = small ? col_act : nullptr; p.ld_col_act = ld_col_act;
    if (!swiglu && !gates_on_input) p.gates = nullptr;
    if (!swiglu && gates_on_input && !p.gates_on_input) p.gates = nullptr;
    p.units = units;
    p.fold = 0;
    p.real_rows = rows;
    p.row_scale = w->row_scale;
    p.hc_hres = hc ? hc->hres : nullptr; p.hc_hpost = hc ? hc->hpost_row : nullptr;
    p.hc_in = hc ? hc->carrier_in : nullptr; p.hc_out = hc ? hc->carrier_out : nullptr;
    p.hc_term = hc ? hc->term : nullptr; p.hc_n = hc ? hc->n_streams : 0;
    p.hc_ld = hc ? (long long)hc->n_streams * ld_out : 0;
    // Small batches: fold the P exact planes into the 8 columns of one MMA (one MMA and one pair
    // of activation loads per tile instead of P of each).  Needs the planes back to back.
    if (n_planes > 1 && rows * n_planes <= 8 && plane_stride == rows * ld_planes) {
        p.fold = n_planes;
        p.rows = rows * n_planes;
        p.n_planes = 1;
    }

    const double avg = (double)w->n_groups / (double)units;   // groups per unit
    const int wpr = avg >= 3.0 ? 4 : (avg >= 1.5 ? 2 : 1);
    cudaStream_t st = (cudaStream_t)stream;
    // Kernel path.  Measured on B200 at the 30B-model shapes (8192 x 43648 / 21824 x 8192, 25%
    // tiles, batch 1..8) the plain path is the fastest of the three or within noise of it, so
    // it is what MORTAR_FLAG_PATH_AUTO runs; the staged and persistent paths run when pinned.
    const int path = flags & MORTAR_FLAG_PATH_MASK;
    const bool persistent_ok = p.n_planes == 1 && p.rows <= 8 && !p.gates && !p.row_act && !p.col_act &&
                               !p.gates_on_input && ps_layout(p.C, (int)p.rows, swiglu).total <= kPsMaxSmem;
    if (persistent_ok && path == MORTAR_FLAG_PATH_PERSISTENT)
        return swiglu ? launch_persistent<true>(p, st) : launch_persistent<false>(p, st);
    const bool bulk = wpr == 4 && path == MORTAR_FLAG_PATH_STAGED;
    return swiglu ? launch_planes<true>(p, wpr, bulk, st) : launch_planes<false>(p, wpr, bulk, st);
}

extern "C" int mortar_linear(const mortar_stream *w, const void *planes, int32_t n_planes,
                             int64_t plane_stride, int64_t ld_planes, int64_t rows, void *out,
                             int32_t out_mode, int32_t n_out_planes, int64_t out_plane_stride,
                             int64_t ld_out, int32_t flags, const float *gates, int64_t ld_gates,
                             int32_t cluster_size, const int32_t *row_act, int64_t ld_row_act,
                             const int32_t *col_act, int64_t ld_col_act, void *stream) {
    if (out_mode == MORTAR_OUT_HC) return MORTAR_ERR_DTYPE;
    return linear_impl(w, planes, n_planes, plane_stride, ld_planes, rows, out, out_mode, n_out_planes,
                       out_plane_stride, ld_out, flags, gates, ld_gates, cluster_size, row_act, ld_row_act,
                       col_act, ld_col_act, nullptr, stream);
}

extern "C" int mortar_linear_hc(const mortar_stream *w, const void *planes, int32_t n_planes,
                                int64_t plane_stride, int64_t ld_planes, int64_t rows,
                                const mortar_hc_post *hc, int64_t ld_stream, int32_t flags,
                                const int32_t *col_act, int64_t ld_col_act, void *stream) {
    if (!hc) return MORTAR_ERR_NULL;
    return linear_impl(w, planes, n_planes, plane_stride, ld_planes, rows, hc->carrier_out, MORTAR_OUT_HC, 0, 0,
                       ld_stream, flags, nullptr, 0, 0, nullptr, 0, col_act, ld_col_act, hc, stream);
}

extern "C" int mortar_route_gather(const float *gates, int64_t rows, int64_t ld_gates, int32_t cluster_size,
                                   int32_t units, int32_t *cnt, int32_t *list, int64_t ld_list, void *stream) {
    if (!gates || !cnt || !list) return MORTAR_ERR_NULL;
    if (rows < 0 || units <= 0 || cluster_size <= 0 || ld_list < rows) return MORTAR_ERR_SHAPE;
    if (rows > 0x7fffffffLL) return MORTAR_ERR_CAPACITY;
    route_gather_kernel<<<(unsigned)((units + 3) / 4), 128, 0, (cudaStream_t)stream>>>(
        gates, ld_gates, (int)rows, cluster_size, units, cnt, list, ld_list);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

extern "C" int mortar_linear_gathered(const mortar_stream *w, const void *planes, int32_t n_planes,
                                      int64_t plane_stride, int64_t ld_planes, int64_t rows, void *out,
                                      int32_t out_mode, int32_t n_out_planes, int64_t out_plane_stride,
                                      int64_t ld_out, int32_t flags, const float *gates, int64_t ld_gates,
                                      int32_t cluster_size, const int32_t *cnt, const int32_t *list,
                                      int64_t ld_list, void *stream) {
    if (!w || !planes || !out || !w->grp_ptr || !gates || !cnt || !list) return MORTAR_ERR_NULL;
    if (w->n_groups > 0 && (!w->grp_codes || !w->grp_cols)) return MORTAR_ERR_NULL;
    if (w->tile_rows <= 0 || (w->tile_rows % 2) || w->tile_cols <= 0 || w->tile_cols > 65534 || rows < 0 ||
        cluster_size <= 0 || ld_list < rows)
        return MORTAR_ERR_SHAPE;
    if (n_planes < 1 || n_planes > 3) return MORTAR_ERR_DTYPE;
    if (out_mode < MORTAR_OUT_F32 || out_mode > MORTAR_OUT_PLANES) return MORTAR_ERR_DTYPE;
    if (out_mode == MORTAR_OUT_PLANES && (n_out_planes < 1 || n_out_planes > 3)) return MORTAR_ERR_DTYPE;
    const int units = w->tile_rows / 2;
    if (ld_planes < (int64_t)w->tile_cols * 16 || ld_out < (int64_t)units * 16) return MORTAR_ERR_SHAPE;
    if (!aligned(planes, 4) || (ld_planes & 1) || (plane_stride & 1)) return MORTAR_ERR_ALIGN;
    if (!aligned(w->grp_codes, 16) || !aligned(w->grp_cols, 16)) return MORTAR_ERR_ALIGN;
    if (flags & MORTAR_FLAG_ACCUMULATE) return MORTAR_ERR_UNSUPPORTED;
    if (rows == 0) return MORTAR_OK;
    if (rows > 0x7fffffffLL) return MORTAR_ERR_CAPACITY;
    LinearParams p;
    p.grp_codes = reinterpret_cast<const uint4 *>(w->grp_codes);
    p.grp_cols = reinterpret_cast<const uint4 *>(w->grp_cols);
    p.grp_ptr = w->grp_ptr;
    p.R = w->tile_rows; p.C = w->tile_cols; p.scale = w->scale;
    p.planes = reinterpret_cast<const uint32_t *>(planes);
    p.plane_stride_w = plane_stride / 2; p.ld_w = ld_planes / 2; p.n_planes = n_planes;
    p.rows = rows;
    p.out = out; p.out_mode = out_mode; p.n_out_planes = n_out_planes;
    p.out_plane_stride = out_plane_stride; p.ld_out = ld_out;
    p.round_bf16 = (flags & MORTAR_FLAG_ROUND_BF16) != 0;
    p.accumulate = 0;
    p.gates = gates; p.ld_gates = ld_gates; p.cluster_size = cluster_size;
    p.gates_on_input = 0;
    p.row_act = nullptr; p.ld_row_act = 0; p.col_act = nullptr; p.ld_col_act = 0;
    p.units = units; p.fold = 0; p.real_rows = rows;
    p.row_scale = nullptr;
    p.hc_hres = p.hc_hpost = p.hc_in = p.hc_term = nullptr; p.hc_out = nullptr; p.hc_n = 0; p.hc_ld = 0;
    const double avg = (double)w->n_groups / (double)units;
    const int wpr = avg >= 3.0 ? 4 : (avg >= 1.5 ? 2 : 1);
    cudaStream_t st = (cudaStream_t)stream;
    if (n_planes == 1) return launch_gather<1>(p, wpr, cnt, list, ld_list, st);
    if (n_planes == 2) return launch_gather<2>(p, wpr, cnt, list, ld_list, st);
    return launch_gather<3>(p, wpr, cnt, list, ld_list, st);
}

extern "C" int mortar_linear_error(int32_t *code, int32_t reset) {
    if (!code) return MORTAR_ERR_NULL;
    int v = 0;
    MORTAR_CUDA_CHECK(cudaMemcpyFromSymbol(&v, g_linear_error, sizeof(int)));
    *code = v;
    if (reset && v != 0) {
        const int zero = 0;
        MORTAR_CUDA_CHECK(cudaMemcpyToSymbol(g_linear_error, &zero, sizeof(int)));
    }
    return MORTAR_OK;
}

extern "C" int mortar_route_flags(const float *gates, int64_t rows, int64_t ld_gates,
                                  const int32_t *row_lo, const int32_t *row_hi, int32_t n_row,
                                  const int32_t *col_lo, const int32_t *col_hi, int32_t n_col,
                                  int32_t *row_act, int64_t ld_row_act, int32_t *col_act,
                                  int64_t ld_col_act, void *stream) {
    if (!gates || !row_lo || !row_hi || !col_lo || !col_hi || !row_act || !col_act) return MORTAR_ERR_NULL;
    if (rows < 0 || n_row < 0 || n_col < 0) return MORTAR_ERR_SHAPE;
    if (rows == 0) return MORTAR_OK;
    if (rows > 0x7fffffffLL) return MORTAR_ERR_CAPACITY;
    route_flags_kernel<<<(unsigned)rows, 128, 0, (cudaStream_t)stream>>>(
        gates, ld_gates, row_lo, row_hi, n_row, col_lo, col_hi, n_col, row_act, ld_row_act, col_act,
        ld_col_act);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

extern "C" int64_t mortar_mlp_workspace_bytes(int64_t rows, int32_t d_model, int32_t d_ff,
                                              int32_t n_planes) {
    if (rows < 0 || d_model <= 0 || d_ff <= 0 || n_planes < 1 || n_planes > 3) return MORTAR_ERR_SHAPE;
    // activation planes of the input and of the hidden layer, then the routing lists of a gated
    // call (per hidden tile row: a count and up to `rows` row numbers)
    return align_up((int64_t)n_planes * rows * d_model * 2, 256) +
           align_up((int64_t)n_planes * rows * d_ff * 2, 256) + align_up((int64_t)(d_ff / 16) * 4, 256) +
           align_up((int64_t)(d_ff / 16) * rows * 4, 256);
}

static int mlp_decode_impl(const mortar_stream *gate_up, const mortar_stream *down,
                           const void *x, int x_dtype, int64_t ldx, int64_t rows,
                           const float *rms_weight, float eps, const float *gates,
                           int64_t ld_gates, int32_t n_clusters, void *y, int y_dtype,
                           int64_t ldy, int32_t n_planes, int32_t flags, void *workspace,
                           int64_t workspace_bytes, const mortar_hc_post *hc, void *stream) {
    if (hc != nullptr) { y = hc->carrier_out; y_dtype = MORTAR_F32; }
    if (!gate_up || !down || !x || !y || !workspace) return MORTAR_ERR_NULL;
    if (x_dtype != MORTAR_F32 && x_dtype != MORTAR_BF16) return MORTAR_ERR_DTYPE;
    if (y_dtype != MORTAR_F32 && y_dtype != MORTAR_BF16) return MORTAR_ERR_DTYPE;
    if (n_planes < 1 || n_planes > 3) return MORTAR_ERR_DTYPE;
    const int d_model = gate_up->tile_cols * 16;
    if (gate_up->tile_rows % 2) return MORTAR_ERR_SHAPE;
    const int d_ff = gate_up->tile_rows * 8;
    if (down->tile_cols * 16 != d_ff || down->tile_rows * 16 != d_model) return MORTAR_ERR_SHAPE;
    if (gates && (n_clusters <= 0 || d_ff % n_clusters)) return MORTAR_ERR_SHAPE;
    if (!aligned(workspace, 256)) return MORTAR_ERR_ALIGN;
    const int64_t need = mortar_mlp_workspace_bytes(rows, d_model, d_ff, n_planes);
    if (need < 0) return (int)need;
    if (workspace_bytes < need) return MORTAR_ERR_CAPACITY;
    if (rows == 0) return MORTAR_OK;

    char *ws = reinterpret_cast<char *>(workspace);
    void *xp = ws;
    void *hp = ws + align_up((int64_t)n_planes * rows * d_model * 2, 256);
    const void *xin = xp;
    int xin_planes = n_planes;
    int64_t xin_stride = rows * (int64_t)d_model, xin_ld = d_model;
    if (x_dtype == MORTAR_BF16 && rms_weight == nullptr && aligned(x, 4) && (ldx % 2) == 0) {
        xin = x; xin_planes = 1; xin_stride = 0; xin_ld = ldx;       // bf16 input is already a plane
    } else {
        int rc = mortar_act_prep(x, x_dtype, rows, d_model, ldx, rms_weight, eps, xp, n_planes,
                                 xin_stride, xin_ld, stream);
        if (rc != MORTAR_OK) return rc;
    }
    const int cs = gates ? d_ff / n_clusters : 0;
    const int rb = flags & MORTAR_FLAG_ROUND_BF16;
    const int h_planes = rb ? 1 : n_planes;
    const int path = flags & MORTAR_FLAG_PATH_MASK;
    int rc;
    if (gates && rows > 8) {
        // routed batch: hidden tile rows run over the rows that activate them only; the rest of the
        // hidden layer is the zero the gate multiply would produce
        char *lp = reinterpret_cast<char *>(hp) + align_up((int64_t)n_planes * rows * d_ff * 2, 256);
        int32_t *cnt = reinterpret_cast<int32_t *>(lp);
        int32_t *list = reinterpret_cast<int32_t *>(lp + align_up((int64_t)(d_ff / 16) * 4, 256));
        MORTAR_CUDA_CHECK(cudaMemsetAsync(hp, 0, (size_t)h_planes * rows * d_ff * 2, (cudaStream_t)stream));
        rc = mortar_route_gather(gates, rows, ld_gates, cs, d_ff / 16, cnt, list, rows, stream);
        if (rc != MORTAR_OK) return rc;
        rc = mortar_linear_gathered(gate_up, xin, xin_planes, xin_stride, xin_ld, rows, hp, MORTAR_OUT_PLANES,
                                    h_planes, rows * (int64_t)d_ff, d_ff, rb, gates, ld_gates, cs, cnt, list,
                                    rows, stream);
    } else {
        rc = mortar_linear(gate_up, xin, xin_planes, xin_stride, xin_ld, rows, hp, MORTAR_OUT_PLANES,
                           h_planes, rows * (int64_t)d_ff, d_ff, MORTAR_FLAG_SWIGLU | rb | path, gates,
                           ld_gates, cs, nullptr, 0, nullptr, 0, stream);
    }
    if (rc != MORTAR_OK) return rc;
    return linear_impl(down, hp, h_planes, rows * (int64_t)d_ff, d_ff, rows, y,
                       y_dtype == MORTAR_F32 ? MORTAR_OUT_F32 : MORTAR_OUT_BF16, 0, 0, ldy,
                       rb | path | (hc ? 0 : (flags & MORTAR_FLAG_ACCUMULATE)) | (gates ? MORTAR_FLAG_GATES_ON_INPUT : 0),
                       gates, ld_gates, cs, nullptr, 0, nullptr, 0, hc, stream);
}

extern "C" int mortar_mlp_decode(const mortar_stream *gate_up, const mortar_stream *down,
                                 const void *x, int x_dtype, int64_t ldx, int64_t rows,
                                 const float *rms_weight, float eps, const float *gates,
                                 int64_t ld_gates, int32_t n_clusters, void *y, int y_dtype,
                                 int64_t ldy, int32_t n_planes, int32_t flags, void *workspace,
                                 int64_t workspace_bytes, void *stream) {
    return mlp_decode_impl(gate_up, down, x, x_dtype, ldx, rows, rms_weight, eps, gates, ld_gates, n_clusters, y,
                           y_dtype, ldy, n_planes, flags, workspace, workspace_bytes, nullptr, stream);
}

extern "C" int mortar_mlp_decode_hc(const mortar_stream *gate_up, const mortar_stream *down,
                                    const void *x, int x_dtype, int64_t ldx, int64_t rows,
                                    const float *rms_weight, float eps, const float *gates,
                                    int64_t ld_gates, int32_t n_clusters, const mortar_hc_post *hc,
                                    int64_t ld_stream, int32_t n_planes, int32_t flags, void *workspace,
                                    int64_t workspace_bytes, void *stream) {
    if (!hc) return MORTAR_ERR_NULL;
    if (flags & (MORTAR_FLAG_ROUND_BF16 | MORTAR_FLAG_ACCUMULATE)) return MORTAR_ERR_UNSUPPORTED;
    return mlp_decode_impl(gate_up, down, x, x_dtype, ldx, rows, rms_weight, eps, gates, ld_gates, n_clusters,
                           hc->carrier_out, MORTAR_F32, ld_stream, n_planes, flags, workspace, workspace_bytes, hc,
                           stream);
}

// ---- MLP application on built-in scratch ---------------------------------------------------
// Scratch for mortar_mlp_decode_static: activation planes of the input and of the hidden
// layer.  It lives in the library image, so every GPU that loads the library holds these
// bytes until the process exits.
#define MORTAR_STATIC_SCRATCH_BYTES (8u << 20)
static __device__ __align__(256) unsigned char g_mlp_static_scratch[MORTAR_STATIC_SCRATCH_BYTES];

namespace {
std::mutex g_static_scratch_mutex;
void *g_static_scratch_ptr[64] = {nullptr};   // device address of the array, per device ordinal
}  // namespace

extern "C" int64_t mortar_mlp_static_scratch_bytes(void) { return (int64_t)MORTAR_STATIC_SCRATCH_BYTES; }

extern "C" int mortar_mlp_decode_static(const mortar_stream *gate_up, const mortar_stream *down,
                                        const void *x, int x_dtype, int64_t ldx, int64_t rows,
                                        const float *rms_weight, float eps, const float *gates,
                                        int64_t ld_gates, int32_t n_clusters, void *y, int y_dtype,
                                        int64_t ldy, int32_t n_planes, int32_t flags, void *stream) {
    if (!gate_up || !down) return MORTAR_ERR_NULL;
    if (rows < 0) return MORTAR_ERR_SHAPE;
    if (n_planes < 1 || n_planes > 3) return MORTAR_ERR_DTYPE;
    const int64_t need = mortar_mlp_workspace_bytes(rows, gate_up->tile_cols * 16, gate_up->tile_rows * 8,
                                                    n_planes);
    if (need < 0) return (int)need;
    if (need > (int64_t)MORTAR_STATIC_SCRATCH_BYTES) return MORTAR_ERR_CAPACITY;   // rows too large for the built-in scratch
    int dev = 0;
    MORTAR_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MORTAR_ERR_CAPACITY;
    void *scratch = nullptr;
    {
        // First call on this device: resolve the device address of the array.  The array's
        // name is only a host-side handle; kernels must be given the address from here.
        std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
        if (g_static_scratch_ptr[dev] == nullptr) {
            void *ptr = nullptr;
            MORTAR_CUDA_CHECK(cudaGetSymbolAddress(&ptr, g_mlp_static_scratch));
            g_static_scratch_ptr[dev] = ptr;
        }
        scratch = g_static_scratch_ptr[dev];
    }
    // Every plane element the two stages read is written earlier in the same call, so nothing
    // in the scratch has to start at zero and stale contents of a previous call are harmless.
    return mortar_mlp_decode(gate_up, down, x, x_dtype, ldx, rows, rms_weight, eps, gates, ld_gates,
                             n_clusters, y, y_dtype, ldy, n_planes, flags, scratch,
                             (int64_t)MORTAR_STATIC_SCRATCH_BYTES, stream);
}
