// Persistent decode of a stack of MLP applications on thread-block clusters.
//
// A cluster of CS CTAs owns one block of 8 activation rows and walks the whole list
//     x <- x + down_i(silu(gate_i(n)) * up_i(n)),  n = rmsnorm_i(x)
// by itself, so blocks of rows never synchronise with each other and nothing but the final
// x leaves the SMs.  Inside a cluster, rank c owns hidden tile rows [cU,(c+1)U) and output
// columns [c*OC,(c+1)*OC): it computes its slice of the hidden layer for the 8 rows (gate and up
// rows of its slice), multiplies it straight into the matching K-slice of the down projection (a
// partial sum over its slice for every output), and PUSHES the partial sums of every rank's
// output columns into that rank's shared memory with one bulk copy per rank (shared memory to
// distributed shared memory, completion counted on the receiver's mbarrier).  Each rank adds the
// CS blocks it received in rank order (deterministic), adds the residual, and pushes its new
// slice of x -- with the slice's sum of squares, so the next RMSNorm needs no reduction pass --
// to every rank the same way.  An application therefore costs two waits on LOCAL mbarriers and no
// cluster-wide barrier; a rank only ever waits for data it is about to read.  The weights of rank
// c for application i+1 (one contiguous blob) stream into shared memory with a bulk copy while
// application i computes.  Arithmetic is the streaming kernel's: ternary tile as the A operand of
// mma.m16n8k16 decoded from 2-bit codes in registers, 8 activation rows as exact bf16 planes as
// the B operand (one accumulator per plane, so the MMAs of a tile are independent), fp32
// accumulation, scale after the sum (morph/kernels/triton/fused_decode_step.py:1441-1459).
//
// Two representations of the fp32 activations: 1..3 bf16 planes (three are exact), or two fp16
// planes (H = true).  fp16 carries 11 significant bits, so two planes leave a residual below 2^-22
// of an element -- the size of an fp32 rounding -- at two thirds of the MMAs and fragment loads.
// Its narrow exponent range is handled by exact power-of-two scaling per activation row: the
// normalised rows have unit RMS by construction (rows that skip the RMSNorm are scaled by the
// power of two next to 1/rms), the hidden rows are scaled so that their largest magnitude lies in
// [2^13, 2^14); the inverse factors are applied to the fp32 sums.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cooperative_groups.h>
#include <cstdint>
#include <mutex>
#include "common.h"
#include "decode.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kWarps = 16;
constexpr int kWarpsPerRow = kWarps / 8;      // warps that share one of the 8 activation rows in the elementwise passes
constexpr int kThreads = kWarps * 32;
constexpr uint32_t kWaitLimit = 1u << 22;

struct StackParams {
    const uint8_t *blobs;
    const int *blob_table;         // [n_layers][CS][4]: gate/up part offset (16-byte units), bytes; down part offset, bytes
    const int *app_layer;          // [n_apps]
    const float *rms;              // [n_layers][d_model] or nullptr
    int n_apps;
    int d_model, d_ff;
    int cs;                        // cluster size
    float *x;
    long long ldx;
    int rows;
    float eps;
    int n_planes;
    int f16;                       // 1: the planes are fp16 (two of them), 0: bf16
    int *status;
    int x_pitch, h_pitch;          // shared-memory row pitch of the plane buffers (bf16 elements)
    int max_a, max_b;              // bytes reserved for the gate/up part and for the down part of a rank's weights
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ void mma_16816_h(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// two fp32 values -> P packed 16-bit pairs (residual split, round to nearest at every level)
template <int P, bool H>
__device__ __forceinline__ void split_pair(float a, float b, uint32_t (&out)[P]) {
#pragma unroll
    for (int pl = 0; pl < P; ++pl) {
        if (H) {
            const __half2 h = __floats2half2_rn(a, b);
            out[pl] = *reinterpret_cast<const uint32_t *>(&h);
            a -= __low2float(h); b -= __high2float(h);
        } else {
            const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            out[pl] = *reinterpret_cast<const uint32_t *>(&h);
            a -= __low2float(h); b -= __high2float(h);
        }
    }
}

// 2^k as a float, k clamped to the normal range
__device__ __forceinline__ float pow2i(int k) {
    k = k < -126 ? -126 : (k > 127 ? 127 : k);
    return __int_as_float((k + 127) << 23);
}

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
// Activation planes keep the 8 element pairs of a 16-column tile in fragment order: pair j sits
// at 32-bit word (j & 3) * 2 + (j >> 2), so the two words a lane feeds to one MMA (pairs t and
// t + 4) are adjacent and come with one 64-bit load.
__device__ __forceinline__ int plane_word(int c) {             // 32-bit word of column c's pair within its row
    const int j = (c & 15) >> 1;
    return (c >> 4) * 8 + (j & 3) * 2 + (j >> 2);
}
__device__ __forceinline__ void lds_bfrag(uint32_t addr, uint32_t &b0, uint32_t &b1) {
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];\n" : "=r"(b0), "=r"(b1) : "r"(addr));
}

// All groups of one tile row of a stream-format matrix held in shared memory, against the 8
// staged activation rows.  Everything is addressed in the shared window (32-bit addresses):
// act[pl] = address of plane pl, this lane's row (lane>>2), word 2*(lane&3) of tile 0.  Every plane has
// its own accumulator (independent MMAs); a group whose last slot is a real tile has no padding
// and runs without per-slot tests, so its loads and MMAs interleave freely.
template <int P, bool H, bool CHECK>
__device__ __forceinline__ void tile_group(const uint4 cw, const uint4 cl, const uint32_t (&act)[P],
                                           float (&accp)[P][4]) {
    const uint32_t cws[4] = {cw.x, cw.y, cw.z, cw.w};
    const uint32_t cls[4] = {cl.x, cl.y, cl.z, cl.w};
    if (!CHECK) {
        // all activation fragments of the group first (their latencies overlap), then the arithmetic
        uint32_t b0[8][P], b1[8][P];
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const uint32_t col = (s & 1) ? (cls[s >> 1] >> 16) : (cls[s >> 1] & 0xffffu);
#pragma unroll
            for (int pl = 0; pl < P; ++pl) lds_bfrag(act[pl] + col * 32u, b0[s][pl], b1[s][pl]);
        }
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            uint32_t af[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                af[i] = H ? mortar_decode_pair_h(cws[s >> 1], (s & 1) * 4 + i) : mortar_decode_pair(cws[s >> 1], (s & 1) * 4 + i);
#pragma unroll
            for (int pl = 0; pl < P; ++pl) {
                if (H) mma_16816_h(accp[pl], af, b0[s][pl], b1[s][pl]);
                else mma_16816(accp[pl], af, b0[s][pl], b1[s][pl]);
            }
        }
        return;
    }
#pragma unroll
    for (int s = 0; s < 8; ++s) {
        const uint32_t col = (s & 1) ? (cls[s >> 1] >> 16) : (cls[s >> 1] & 0xffffu);
        if (col != 0xffffu) {                                   // padding slots end a row
            uint32_t af[4];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                af[i] = H ? mortar_decode_pair_h(cws[s >> 1], (s & 1) * 4 + i) : mortar_decode_pair(cws[s >> 1], (s & 1) * 4 + i);
            uint32_t b0[P], b1[P];
#pragma unroll
            for (int pl = 0; pl < P; ++pl) lds_bfrag(act[pl] + col * 32u, b0[pl], b1[pl]);
#pragma unroll
            for (int pl = 0; pl < P; ++pl) {
                if (H) mma_16816_h(accp[pl], af, b0[pl], b1[pl]);
                else mma_16816(accp[pl], af, b0[pl], b1[pl]);
            }
        }
    }
}

template <int P, bool H>
__device__ __forceinline__ void tile_row(uint32_t grp_ptr, uint32_t cols, uint32_t codes, int trow,
                                         const uint32_t (&act)[P], int lane, float (&acc)[4]) {
    int gbeg, gend;
    asm volatile("ld.shared.u32 %0, [%2];\n\tld.shared.u32 %1, [%2+4];\n" : "=r"(gbeg), "=r"(gend) : "r"(grp_ptr + 4u * trow));
    uint32_t caddr = codes + (uint32_t)(gbeg * 32 + lane) * 16u;
    uint32_t laddr = cols + (uint32_t)gbeg * 16u;
    float accp[P][4];
#pragma unroll
    for (int pl = 0; pl < P; ++pl)
#pragma unroll
        for (int i = 0; i < 4; ++i) accp[pl][i] = 0.f;
    for (int grp = gbeg; grp < gend; ++grp, caddr += 512u, laddr += 16u) {
        const uint4 cw = lds128(caddr);
        const uint4 cl = lds128(laddr);
        if ((cl.w >> 16) != 0xffffu) tile_group<P, H, false>(cw, cl, act, accp);
        else tile_group<P, H, true>(cw, cl, act, accp);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float v = accp[0][i];
#pragma unroll
        for (int pl = 1; pl < P; ++pl) v += accp[pl][i];
        acc[i] += v;
    }
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

// Per-phase cycle accounting for profiling builds (-DMORTAR_STACK_TIMING): thread 0 of CTA 0 sums the
// cycles between the phase boundaries of every application into g_stack_ticks.
#ifdef MORTAR_STACK_TIMING
__device__ unsigned long long g_stack_ticks[16];
#define ST_DECL long long st_prev = clock64()
#define ST_ACC(i) do { if (blockIdx.x == 0 && threadIdx.x == 0) { const long long n_ = clock64(); \
        atomicAdd(&g_stack_ticks[i], (unsigned long long)(n_ - st_prev)); st_prev = n_; } } while (0)
#else
#define ST_DECL
#define ST_ACC(i)
#endif

struct SmemLayout {
    int xs, xp, hp, gu, recv, xsend, wbuf, bars, total;   // byte offsets
};

__host__ __device__ inline int align_up_i(int v, int a) { return (v + a - 1) / a * a; }

// xs holds the residual rows rank-major: block q = [8 rows][OC columns] of rank q's output columns
// followed by the 8 sums of squares of those row slices -- the unit one rank pushes to its peers.
__host__ __device__ inline int xs_block_floats(int d_model, int cs) { return 8 * (d_model / cs) + 8; }

__host__ __device__ inline SmemLayout smem_layout(int d_model, int d_ff, int cs, int n_planes, int f16, int x_pitch,
                                                  int h_pitch, int max_a, int max_b) {
    SmemLayout L;
    int off = 0;
    L.xs = off; off += cs * xs_block_floats(d_model, cs) * 4;
    L.xp = off;                                   // planes of the normalised rows; reused for the outgoing partial sums
    const int xp_bytes = n_planes * 8 * x_pitch * 2, ysend_bytes = cs * 8 * (d_model / cs + 4) * 4;
    off += align_up_i(xp_bytes > ysend_bytes ? xp_bytes : ysend_bytes, 16);
    L.hp = off; off += align_up_i(n_planes * 8 * h_pitch * 2, 16);
    L.gu = off;                                   // gate and up sums of the hidden slice, fp32: when a rank has fewer
    // hidden tile rows than warps; with fp16 planes always (the fp32 hidden rows wait there for their scale)
    if (f16 || d_ff / 16 / cs < kWarps) off += 8 * 2 * (d_ff / cs) * 4;
    L.recv = off; off += cs * 8 * (d_model / cs + 4) * 4;   // partial sums of this rank's columns, one block per source rank
    L.xsend = off; off += xs_block_floats(d_model, cs) * 4;
    off = align_up_i(off, 128);
    L.wbuf = off; off += max_a + max_b;           // one buffer per part: a part is refilled as soon as its stage is over
    L.bars = off; off += 32 + 64;                 // 4 mbarriers, 8 row factors of the x planes, 8 row maxima of the hidden rows
    L.total = off;
    return L;
}

__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, int rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(local_addr), "r"(rank));
    return r;
}

// shared memory of this CTA -> shared memory of a CTA of the cluster; the bytes are counted on
// the RECEIVER's mbarrier (both destination addresses are cluster addresses of the same CTA)
__device__ __forceinline__ void push_bulk(uint32_t dst_cluster, uint32_t src_local, uint32_t bytes, uint32_t bar_cluster) {
    asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(dst_cluster), "r"(src_local), "r"(bytes), "r"(bar_cluster) : "memory");
}

template <int P, bool H>
__global__ void __launch_bounds__(kThreads, 1) stack_decode_kernel(const StackParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int cs = p.cs;
    const SmemLayout L = smem_layout(p.d_model, p.d_ff, cs, p.n_planes, p.f16, p.x_pitch, p.h_pitch, p.max_a, p.max_b);
    float *xs = reinterpret_cast<float *>(smem + L.xs);
    uint16_t *xp = reinterpret_cast<uint16_t *>(smem + L.xp);       // planes: bf16 or fp16 bit patterns
    float *ysend = reinterpret_cast<float *>(smem + L.xp);
    uint16_t *hp = reinterpret_cast<uint16_t *>(smem + L.hp);
    float *gu_out = reinterpret_cast<float *>(smem + L.gu);
    float *recv = reinterpret_cast<float *>(smem + L.recv);
    float *xsend = reinterpret_cast<float *>(smem + L.xsend);
    uint8_t *wbuf = smem + L.wbuf;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L.bars);     // [0]: gate/up weights, [1]: down weights; [2]: partial sums; [3]: x slices
    float *xun = reinterpret_cast<float *>(smem + L.bars + 32);       // per row: factor that undoes the scaling of the x planes
    uint32_t *hmax = reinterpret_cast<uint32_t *>(smem + L.bars + 64); // per row: bits of the largest |hidden| (fp16 planes)

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = (int)(blockIdx.x / cs) * 8;                 // this cluster's block of rows
    const int D = p.d_model, OC = D / cs;                         // output columns owned by a rank
    const int U = p.d_ff / 16 / cs;                               // hidden tile rows owned by a rank
    const int RD = D / 16, TR = OC / 16;                          // output tile rows: all, per rank
    const int xplane_w = 8 * p.x_pitch / 2, hplane_w = 8 * p.h_pitch / 2;
    const int blk = xs_block_floats(D, cs);
    // partial-sum blocks use a row pitch of OC + 4 floats: the four row pairs a warp stores at once
    // then fall into different banks
    const int OCP = OC + 4;
    const uint32_t part_bytes = (uint32_t)(8 * OCP * 4), blk_bytes = (uint32_t)(blk * 4);
    const uint32_t pbar = smem_u32(&bars[2]), xbar = smem_u32(&bars[3]);

    auto prefetch = [&](int app, int part) {
        // one bulk copy of part `part` (0 = gate/up, 1 = down) of this rank's weights for application `app`
        const int layer = p.app_layer[app];
        const int *ent = p.blob_table + ((long long)layer * cs + rank) * 4 + part * 2;
        const uint32_t bytes = (uint32_t)ent[1];
        const uint32_t bar = smem_u32(&bars[part]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
            ::"r"(smem_u32(wbuf + (part ? p.max_a : 0))), "l"(p.blobs + (size_t)ent[0] * 16), "r"(bytes), "r"(bar)
            : "memory");
    };
    auto expect = [&](uint32_t bar, uint32_t bytes) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
    };
    // Bounded wait on a local mbarrier phase.  On expiry the status word is set and the walk goes
    // on (with undefined numbers): every rank still sends what its peers wait for and reaches the
    // final cluster barrier.
    auto wait = [&](uint32_t bar, uint32_t parity) {
        for (uint32_t i = 0; i < kWaitLimit; ++i)
            if (mbar_try_wait(bar, parity)) return;
        if (lane == 0) atomicExch(p.status, 1);
    };

    // Both weight buffers start as zeros: a blob of zeros describes tile rows without groups, so if
    // a copy should ever fail to arrive (the bounded wait reports it) the walk over the
    // buffer stays inside it instead of following uninitialised offsets.
    for (int i = threadIdx.x; i < (p.max_a + p.max_b) / 16; i += kThreads)
        reinterpret_cast<uint4 *>(wbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
    // this rank's slice of the residual rows (rows past the batch are zero) and its sums of squares
    for (int e = threadIdx.x; e < 8 * OC; e += kThreads) {
        const int r = e / OC, cl = e - r * OC;
        xsend[e] = (row0 + r < p.rows) ? p.x[(long long)(row0 + r) * p.ldx + rank * OC + cl] : 0.f;
    }
    __syncthreads();
    if (warp < 8) {
        float ss = 0.f;
        for (int cl = lane; cl < OC; cl += 32) { const float v = xsend[warp * OC + cl]; ss += v * v; }
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (lane == 0) xsend[8 * OC + warp] = ss;
    }
    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // generic writes before the bulk copies read them
    if (threadIdx.x == 0) {
        for (int i = 0; i < 4; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&bars[i])));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        expect(pbar, part_bytes * cs);                             // phase 0 of both exchange barriers
        expect(xbar, blk_bytes * cs);
        if (p.n_apps > 0) { prefetch(0, 0); prefetch(0, 1); }
    }
    __syncthreads();
    cluster.sync();          // every CTA of the cluster is resident, its barriers armed, before any push
    if (warp == 0 && lane < cs)
        push_bulk(map_to_rank(smem_u32(xs + rank * blk), lane), smem_u32(xsend), blk_bytes, map_to_rank(xbar, lane));

    ST_DECL;
    for (int a = 0; a < p.n_apps; ++a) {
        ST_ACC(0);
        // ---- gate/up weights of this application (requested when the previous application's
        //      gate/up stage ended) ----
        wait(smem_u32(&bars[0]), a & 1);
        ST_ACC(1);
        // part header: int32 {n_groups, offsets of grp_ptr, grp_cols, grp_codes, scale bits, bytes,
        // offset of an fp32[d_model] rmsnorm weight or 0, 0}
        const uint8_t *part_a = wbuf, *part_b = wbuf + p.max_a;
        const int *ha = reinterpret_cast<const int *>(part_a);
        const uint32_t gu_ptr = smem_u32(part_a) + ha[1], gu_cols = smem_u32(part_a) + ha[2], gu_codes = smem_u32(part_a) + ha[3];
        const float scale_gu = __int_as_float(ha[4]);
        // rmsnorm weight of this application: the copy inside the weights when the packer put one
        // there, else the caller's [n_layers][d_model] array, else no normalisation
        const float *rms_w = ha[6] ? reinterpret_cast<const float *>(part_a + ha[6])
                                   : (p.rms != nullptr ? p.rms + (size_t)p.app_layer[a] * D : nullptr);

        // this thread's norm weights, requested before the wait so their latency hides behind it
        // (they come from global memory unless the blob carries a copy)
        constexpr int kWPre = 2;
        constexpr int kRowStep = kWarpsPerRow * 128;             // columns one sweep of a row's warps covers
        float4 wpre[kWPre];
        if (rms_w != nullptr) {
#pragma unroll
            for (int k = 0; k < kWPre; ++k) {
                const int c = (warp % kWarpsPerRow) * 128 + lane * 4 + k * kRowStep;
                if (c < D) wpre[k] = *reinterpret_cast<const float4 *>(rms_w + c);
            }
        }

        // ---- the residual rows (every rank's slice) have arrived; arm the barrier's next phase ----
        wait(xbar, a & 1);
        if (threadIdx.x == 0) expect(xbar, blk_bytes * cs);
        ST_ACC(2);

        // ---- n = rmsnorm(x) as exact bf16 planes (kWarpsPerRow warps per row) ----
        {
            const int row = warp / kWarpsPerRow, part = warp % kWarpsPerRow;
            float inv = 1.f, undo = 1.f;
            if (rms_w != nullptr || H) {
                float ss = 0.f;
                for (int q = 0; q < cs; ++q) ss += xs[q * blk + 8 * OC + row];      // rank order: same sum in every rank
                if (rms_w != nullptr) {
                    inv = 1.f / sqrtf(ss / (float)D + p.eps);
                } else if (ss > 0.f) {
                    // fp16 planes without a norm: bring the row to unit RMS with the power of two below 1/rms
                    const int eb = (__float_as_int(rsqrtf(ss / (float)D)) >> 23) & 0xff;
                    inv = pow2i(eb - 127);
                    undo = pow2i(127 - eb);
                }
            }
            if (part == 0 && lane == 0) xun[row] = undo;
            if (H && threadIdx.x < 8) hmax[threadIdx.x] = 0u;
            const float inv_oc = 1.f / (float)OC;
            auto plane_split = [&](int c, const float4 wv) {
                const int q = (int)(((float)c + 0.5f) * inv_oc);                   // c / OC for these small integers
                const float4 v = *reinterpret_cast<const float4 *>(xs + q * blk + row * OC + (c - q * OC));
                float vv[4] = {v.x, v.y, v.z, v.w};
                if (rms_w != nullptr) {
                    vv[0] = (vv[0] * inv) * wv.x; vv[1] = (vv[1] * inv) * wv.y;
                    vv[2] = (vv[2] * inv) * wv.z; vv[3] = (vv[3] * inv) * wv.w;
                } else if (H) {
                    vv[0] *= inv; vv[1] *= inv; vv[2] *= inv; vv[3] *= inv;
                }
                // packed conversions (two values per instruction, off the conversion unit)
                uint32_t lo[P], hi[P];
                split_pair<P, H>(vv[0], vv[1], lo);
                split_pair<P, H>(vv[2], vv[3], hi);
                uint32_t *o = reinterpret_cast<uint32_t *>(xp + row * p.x_pitch) + plane_word(c);
#pragma unroll
                for (int pl = 0; pl < P; ++pl) {                // pairs (c, c+1) and (c+2, c+3): two words apart
                    o[pl * xplane_w] = lo[pl];
                    o[pl * xplane_w + 2] = hi[pl];
                }
            };
#pragma unroll
            for (int k = 0; k < kWPre; ++k) {
                const int c = part * 128 + lane * 4 + k * kRowStep;
                if (c < D) plane_split(c, wpre[k]);
            }
            for (int c = part * 128 + lane * 4 + kWPre * kRowStep; c < D; c += kRowStep)
                plane_split(c, rms_w != nullptr ? *reinterpret_cast<const float4 *>(rms_w + c) : make_float4(1.f, 1.f, 1.f, 1.f));
        }
        __syncthreads();
        ST_ACC(3);

        // ---- hidden slice: gate and up sums of this rank's 2U tile rows, one row per warp turn ----
        {
            uint32_t act[P];
#pragma unroll
            for (int pl = 0; pl < P; ++pl)
                act[pl] = smem_u32(xp) + (uint32_t)(pl * xplane_w + g * (p.x_pitch / 2) + 2 * t) * 4u;
            const int W = 2 * U * 16;                            // gate columns then up columns
            const int HW = U * 16;
            // the matrix scale times the factor that undoes the row's plane scaling (rows 2t, 2t+1)
            const float sg[2] = {scale_gu * xun[2 * t], scale_gu * xun[2 * t + 1]};
            // fp16 planes: the fp32 hidden rows wait in shared memory (row pitch hp32) for the row maxima
            const int hp32 = U >= kWarps ? HW + 4 : W;
            if (U >= kWarps) {
                // enough hidden tile rows for every warp: one warp computes the gate and the up
                // tile row of a hidden tile row and applies SwiGLU in registers
                for (int hrow = warp; hrow < U; hrow += kWarps) {
                    float ag[4] = {0.f, 0.f, 0.f, 0.f}, au[4] = {0.f, 0.f, 0.f, 0.f};
                    tile_row<P, H>(gu_ptr, gu_cols, gu_codes, hrow, act, lane, ag);
                    tile_row<P, H>(gu_ptr, gu_cols, gu_codes, U + hrow, act, lane, au);
                    float mx[2] = {0.f, 0.f};
#pragma unroll
                    for (int i = 0; i < 4; i += 2) {             // (neuron g + 8*(i>>1), rows 2t and 2t+1)
                        float hv[2];
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
                            const float gv = sg[k] * ag[i + k], uv = sg[k] * au[i + k];
                            hv[k] = gv * __fdividef(1.f, 1.f + __expf(-gv)) * uv;
                        }
                        const int col = hrow * 16 + g + 8 * (i >> 1);
                        if (H) {
                            gu_out[(2 * t) * hp32 + col] = hv[0];
                            gu_out[(2 * t + 1) * hp32 + col] = hv[1];
                            mx[0] = fmaxf(mx[0], fabsf(hv[0])); mx[1] = fmaxf(mx[1], fabsf(hv[1]));
                        } else {
                            uint32_t pr[P];
                            split_pair<P, H>(hv[0], hv[1], pr);
                            uint16_t *o = hp + (2 * t) * p.h_pitch + plane_word(col) * 2 + (col & 1);
#pragma unroll
                            for (int pl = 0; pl < P; ++pl) {
                                o[(size_t)pl * 8 * p.h_pitch] = (uint16_t)(pr[pl] & 0xffffu);
                                o[(size_t)pl * 8 * p.h_pitch + p.h_pitch] = (uint16_t)(pr[pl] >> 16);
                            }
                        }
                    }
                    if (H) {
                        // largest |hidden| of rows 2t and 2t+1 over this tile row's 16 neurons (lanes of equal t)
#pragma unroll
                        for (int k = 0; k < 2; ++k) {
#pragma unroll
                            for (int o = 4; o < 32; o <<= 1) mx[k] = fmaxf(mx[k], __shfl_xor_sync(0xffffffffu, mx[k], o));
                            if (g == 0) atomicMax(&hmax[2 * t + k], __float_as_uint(mx[k]));
                        }
                    }
                }
            } else {
                for (int trow = warp; trow < 2 * U; trow += kWarps) {
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    tile_row<P, H>(gu_ptr, gu_cols, gu_codes, trow, act, lane, acc);
#pragma unroll
                    for (int i = 0; i < 4; ++i)                  // (neuron g + 8*(i>>1), row 2t + (i&1))
                        gu_out[(2 * t + (i & 1)) * W + trow * 16 + g + 8 * (i >> 1)] = sg[i & 1] * acc[i];
                }
                __syncthreads();
                // silu(gate) * up -> exact bf16 planes of the hidden slice
                const int r = warp / kWarpsPerRow;               // kWarpsPerRow warps per activation row
                for (int c = (warp % kWarpsPerRow) * 32 + lane; c < HW; c += kWarpsPerRow * 32) {
                    const float gv = gu_out[r * W + c], uv = gu_out[r * W + HW + c];
                    float hv = gv * __fdividef(1.f, 1.f + __expf(-gv)) * uv;
                    if (H) {
                        gu_out[r * W + c] = hv;                   // in place of the gate sum this thread just read
                        hv = fabsf(hv);
#pragma unroll
                        for (int o = 1; o < 32; o <<= 1) hv = fmaxf(hv, __shfl_xor_sync(0xffffffffu, hv, o));
                        if (lane == 0) atomicMax(&hmax[r], __float_as_uint(hv));
                    } else {
                        uint16_t *o = hp + r * p.h_pitch + plane_word(c) * 2 + (c & 1);
#pragma unroll
                        for (int pl = 0; pl < P; ++pl) {
                            const __nv_bfloat16 hb = __float2bfloat16_rn(hv);
                            o[(size_t)pl * 8 * p.h_pitch] = __bfloat16_as_ushort(hb);
                            hv -= __bfloat162float(hb);
                        }
                    }
                }
            }
            if (H) {
                // every hidden row scaled so that its largest magnitude lies in [2^13, 2^14), then split
                __syncthreads();
                const int r = warp / kWarpsPerRow;
                const uint32_t mb = hmax[r];
                const float sc = mb ? pow2i(13 + 127 - (int)(mb >> 23)) : 1.f;
                for (int c = (warp % kWarpsPerRow) * 64 + lane * 2; c < HW; c += kWarpsPerRow * 64) {
                    const float2 v = *reinterpret_cast<const float2 *>(gu_out + r * hp32 + c);
                    uint32_t pr[P];
                    split_pair<P, H>(v.x * sc, v.y * sc, pr);
#pragma unroll
                    for (int pl = 0; pl < P; ++pl)
                        reinterpret_cast<uint32_t *>(hp + r * p.h_pitch)[pl * hplane_w + plane_word(c)] = pr[pl];
                }
            }
        }
        __syncthreads();
        if (threadIdx.x == 0 && a + 1 < p.n_apps) prefetch(a + 1, 0);     // the gate/up buffer is free again
        wait(smem_u32(&bars[1]), a & 1);                                    // down weights of this application
        const int *hb = reinterpret_cast<const int *>(part_b);
        const uint32_t dn_ptr = smem_u32(part_b) + hb[1], dn_cols = smem_u32(part_b) + hb[2], dn_codes = smem_u32(part_b) + hb[3];
        const float scale_dn = __int_as_float(hb[4]);
        ST_ACC(4);

        // ---- partial down projection over this rank's hidden slice, for every output; the sums of
        //      output tile row trow go to the block of the rank that owns those columns ----
        {
            uint32_t act[P];
#pragma unroll
            for (int pl = 0; pl < P; ++pl)
                act[pl] = smem_u32(hp) + (uint32_t)(pl * hplane_w + g * (p.h_pitch / 2) + 2 * t) * 4u;
            float sd[2] = {scale_dn, scale_dn};                  // times the factor that undoes the hidden rows' scaling
            if (H) {
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const uint32_t mb = hmax[2 * t + k];
                    if (mb) sd[k] = scale_dn * pow2i((int)(mb >> 23) - 127 - 13);
                }
            }
            for (int trow = warp; trow < RD; trow += kWarps) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                tile_row<P, H>(dn_ptr, dn_cols, dn_codes, trow, act, lane, acc);
                const int q = trow / TR, cl0 = (trow - q * TR) * 16;
                float *dst = ysend + (size_t)q * 8 * OCP + cl0;
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    dst[(2 * t + (i & 1)) * OCP + g + 8 * (i >> 1)] = sd[i & 1] * acc[i];
            }
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncthreads();
        if (warp == 0 && lane < cs)
            push_bulk(map_to_rank(smem_u32(recv + (size_t)rank * 8 * OCP), lane), smem_u32(ysend + (size_t)lane * 8 * OCP),
                      part_bytes, map_to_rank(pbar, lane));
        if (threadIdx.x == 32 && a + 1 < p.n_apps) prefetch(a + 1, 1);    // the down buffer is free again

        ST_ACC(5);
        // ---- the partial sums of this rank's columns have arrived from every rank ----
        wait(pbar, a & 1);
        ST_ACC(6);
        if (threadIdx.x == 0) expect(pbar, part_bytes * cs);
        // new residual slice = old slice + partial sums in rank order; one warp per row
        if (warp < 8) {
            const int r = warp;
            float ss = 0.f;
            for (int cl = lane; cl < OC; cl += 32) {
                float v = xs[rank * blk + r * OC + cl];
                for (int q = 0; q < cs; ++q) v += recv[((size_t)q * 8 + r) * OCP + cl];
                xsend[r * OC + cl] = v;
                ss += v * v;
            }
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) xsend[8 * OC + r] = ss;
        }
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
        __syncthreads();
        if (warp == 0 && lane < cs)
            push_bulk(map_to_rank(smem_u32(xs + rank * blk), lane), smem_u32(xsend), blk_bytes, map_to_rank(xbar, lane));
        ST_ACC(7);
    }

    // this rank writes its column slice of the final rows (its own latest slice)
    for (int e = threadIdx.x; e < 8 * OC; e += kThreads) {
        const int r = e / OC, cl = e - r * OC;
        if (row0 + r < p.rows) p.x[(long long)(row0 + r) * p.ldx + rank * OC + cl] = xsend[e];
    }
    // every slice pushed to this CTA has landed before it may exit; after the cluster barrier no
    // peer still reads this CTA's shared memory either
    wait(xbar, p.n_apps & 1);
    cluster.sync();
}

inline int pitch_for(int features) {
    // row pitch (bf16 elements) whose 32-bit word count is 8 mod 32: the 4 rows x 4 lanes of each
    // half of a 64-bit B-fragment load then hit 32 different banks
    const int words = features / 2;
    const int pad = ((8 - words % 32) % 32 + 32) % 32;
    return (words + pad) * 2;
}

}  // namespace

#ifdef MORTAR_STACK_TIMING
extern "C" int mortar_stack_ticks(unsigned long long *out) {
    MORTAR_CUDA_CHECK(cudaMemcpyFromSymbol(out, g_stack_ticks, sizeof(unsigned long long) * 16));
    static const unsigned long long zeros[16] = {0};
    MORTAR_CUDA_CHECK(cudaMemcpyToSymbol(g_stack_ticks, zeros, sizeof(zeros)));
    return MORTAR_OK;
}
#endif

extern "C" int mortar_stack_decode(const void *blobs, const int32_t *blob_table, const int32_t *app_layer,
                                   const float *rms_weights, int32_t n_apps, int32_t n_layers,
                                   int32_t d_model, int32_t d_ff, int32_t max_gate_up_bytes, int32_t max_down_bytes,
                                   int32_t cluster_size, float *x, int64_t ldx, int64_t rows, float eps,
                                   int32_t n_planes, int32_t *status, void *stream) {
    if (!blobs || !blob_table || !app_layer || !x || !status) return MORTAR_ERR_NULL;
    if (n_layers <= 0) return MORTAR_ERR_SHAPE;
    if (rms_weights && (reinterpret_cast<uintptr_t>(rms_weights) % 16)) return MORTAR_ERR_ALIGN;
    if (n_apps < 0 || d_model <= 0 || d_ff <= 0 || d_model % 16 || d_ff % 16 || rows < 0 || ldx < d_model)
        return MORTAR_ERR_SHAPE;
    if (cluster_size != 8 && cluster_size != 16) return MORTAR_ERR_SHAPE;
    if ((d_ff / 16) % cluster_size || d_model % (16 * cluster_size)) return MORTAR_ERR_SHAPE;
    const int f16 = n_planes == MORTAR_PLANES_HALF2 ? 1 : 0;
    if (f16) n_planes = 2;
    if (n_planes < 1 || n_planes > 3) return MORTAR_ERR_DTYPE;
    if ((reinterpret_cast<uintptr_t>(blobs) % 16) || (reinterpret_cast<uintptr_t>(x) % 16) || (ldx % 4) ||
        (max_gate_up_bytes % 128) || (max_down_bytes % 128) || max_gate_up_bytes < 128 || max_down_bytes < 128)
        return MORTAR_ERR_ALIGN;
    if (rows == 0 || n_apps == 0) return MORTAR_OK;
    if (rows > 8 * 65535LL / cluster_size) return MORTAR_ERR_CAPACITY;

    int dev = 0;
    MORTAR_CUDA_CHECK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return MORTAR_ERR_CAPACITY;
    static int smem_optin[64] = {0};
    static std::mutex init_mutex;
    int smem_limit = 0;
    {
    std::lock_guard<std::mutex> lock(init_mutex);
    if (smem_optin[dev] == 0) {
        int v = 0;
        MORTAR_CUDA_CHECK(cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        v -= 256;                                      // room for the kernel's few static shared bytes
        void (*kernels[4])(const StackParams) = {stack_decode_kernel<1, false>, stack_decode_kernel<2, false>,
                                                 stack_decode_kernel<3, false>, stack_decode_kernel<2, true>};
        for (auto k : kernels) {
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, v));
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(k, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
        }
        smem_optin[dev] = v;
    }
    smem_limit = smem_optin[dev];
    }
    StackParams p;
    p.blobs = reinterpret_cast<const uint8_t *>(blobs);
    p.blob_table = blob_table; p.app_layer = app_layer; p.rms = rms_weights;
    p.n_apps = n_apps; p.d_model = d_model; p.d_ff = d_ff; p.cs = cluster_size;
    p.x = x; p.ldx = ldx; p.rows = (int)rows; p.eps = eps; p.n_planes = n_planes; p.f16 = f16; p.status = status;
    p.x_pitch = pitch_for(d_model);
    p.h_pitch = pitch_for(d_ff / cluster_size);
    p.max_a = max_gate_up_bytes; p.max_b = max_down_bytes;
    const SmemLayout L = smem_layout(d_model, d_ff, cluster_size, n_planes, f16, p.x_pitch, p.h_pitch, max_gate_up_bytes, max_down_bytes);
    if (L.total > smem_limit) return MORTAR_ERR_CAPACITY;   // a rank's share does not fit shared memory

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(((rows + 7) / 8) * cluster_size));
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = (size_t)L.total;
    cfg.stream = (cudaStream_t)stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)cluster_size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (f16) MORTAR_CUDA_CHECK(cudaLaunchKernelEx(&cfg, stack_decode_kernel<2, true>, p));
    else if (n_planes == 1) MORTAR_CUDA_CHECK(cudaLaunchKernelEx(&cfg, stack_decode_kernel<1, false>, p));
    else if (n_planes == 2) MORTAR_CUDA_CHECK(cudaLaunchKernelEx(&cfg, stack_decode_kernel<2, false>, p));
    else MORTAR_CUDA_CHECK(cudaLaunchKernelEx(&cfg, stack_decode_kernel<3, false>, p));
    return MORTAR_OK;
}
