// Persistent decode of a stack of MLP applications on thread-block clusters.
//
// A cluster of CS CTAs owns one block of 8 activation rows and walks the whole list
//     x <- x + down_i(silu(gate_i(n)) * up_i(n)),  n = rmsnorm_i(x)
// by itself, so blocks of rows never synchronise with each other and nothing but the final
// x leaves the SMs.  Inside a cluster, rank c owns hidden tile rows [cU,(c+1)U): it computes
// that slice of the hidden layer for the 8 rows (gate and up rows of its slice), multiplies
// it straight into the matching K-slice of the down projection (a partial sum over its slice
// for every output), and the ranks combine the partial sums through distributed shared
// memory in rank order (deterministic).  Two cluster barriers per application.  The weights
// of rank c for application i+1 (one contiguous blob) stream into shared memory with a bulk
// copy while application i computes.  Arithmetic is the streaming kernel's: ternary tile as
// the A operand of mma.m16n8k16 decoded from 2-bit codes in registers, 8 activation rows as
// exact bf16 planes as the B operand, fp32 accumulation, scale after the sum
// (morph/kernels/triton/fused_decode_step.py:1441-1459).
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cooperative_groups.h>
#include <cstdint>
#include <mutex>
#include "common.h"
#include "decode.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr uint32_t kWaitLimit = 1u << 22;

struct StackParams {
    const uint8_t *blobs;
    const int *blob_table;         // [n_layers][CS][2]
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
    int *status;
    int x_pitch, h_pitch;          // shared-memory row pitch of the plane buffers (bf16 elements)
    int max_blob;                  // bytes reserved per weight buffer
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

__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];\n" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void lds_bfrag(uint32_t addr, uint32_t &b0, uint32_t &b1) {
    asm volatile("ld.shared.u32 %0, [%2];\n\tld.shared.u32 %1, [%2+16];\n" : "=r"(b0), "=r"(b1) : "r"(addr));
}

// All groups of one tile row of a stream-format matrix held in shared memory, against the 8
// staged activation rows.  Everything is addressed in the shared window (32-bit addresses):
// act[pl] = address of plane pl, this lane's row (lane>>2), element 2*(lane&3).
template <int P>
__device__ __forceinline__ void tile_row(uint32_t grp_ptr, uint32_t cols, uint32_t codes, int trow,
                                         const uint32_t (&act)[P], int lane, float (&acc)[4]) {
    int gbeg, gend;
    asm volatile("ld.shared.u32 %0, [%2];\n\tld.shared.u32 %1, [%2+4];\n" : "=r"(gbeg), "=r"(gend) : "r"(grp_ptr + 4u * trow));
    uint32_t caddr = codes + (uint32_t)(gbeg * 32 + lane) * 16u;
    uint32_t laddr = cols + (uint32_t)gbeg * 16u;
    for (int grp = gbeg; grp < gend; ++grp, caddr += 512u, laddr += 16u) {
        const uint4 cw = lds128(caddr);
        const uint4 cl = lds128(laddr);
        const uint32_t cws[4] = {cw.x, cw.y, cw.z, cw.w};
        const uint32_t cls[4] = {cl.x, cl.y, cl.z, cl.w};
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const uint32_t col = (s & 1) ? (cls[s >> 1] >> 16) : (cls[s >> 1] & 0xffffu);
            if (col != 0xffffu) {                               // padding slots end a row
                uint32_t af[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) af[i] = mortar_decode_pair(cws[s >> 1], (s & 1) * 4 + i);
                uint32_t b0[P], b1[P];
#pragma unroll
                for (int pl = 0; pl < P; ++pl) lds_bfrag(act[pl] + col * 32u, b0[pl], b1[pl]);
#pragma unroll
                for (int pl = 0; pl < P; ++pl) mma_16816(acc, af, b0[pl], b1[pl]);
            }
        }
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

struct SmemLayout {
    int xs, xp, hp, gu, xnew, wbuf, bars, total;   // byte offsets
};

__host__ __device__ inline int align_up_i(int v, int a) { return (v + a - 1) / a * a; }

__host__ __device__ inline SmemLayout smem_layout(int d_model, int d_ff, int cs, int n_planes, int x_pitch,
                                                  int h_pitch, int max_blob) {
    SmemLayout L;
    int off = 0;
    L.xs = off; off += 8 * d_model * 4;
    L.xp = off;                                   // planes of the normalised rows; reused for the partial sums
    const int xp_bytes = n_planes * 8 * x_pitch * 2, ypart_bytes = 8 * d_model * 4;
    off += align_up_i(xp_bytes > ypart_bytes ? xp_bytes : ypart_bytes, 16);
    L.hp = off; off += align_up_i(n_planes * 8 * h_pitch * 2, 16);
    L.gu = off; off += 8 * 2 * (d_ff / cs) * 4;       // gate and up sums of the hidden slice, fp32
    L.xnew = off; off += 2 * 8 * (d_model / cs) * 4;
    off = align_up_i(off, 128);
    L.wbuf = off; off += 2 * max_blob;
    L.bars = off; off += 16;
    L.total = off;
    return L;
}

template <int P>
__global__ void __launch_bounds__(kThreads, 1) stack_decode_kernel(const StackParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int rank = (int)cluster.block_rank();
    const int cs = p.cs;
    const SmemLayout L = smem_layout(p.d_model, p.d_ff, cs, p.n_planes, p.x_pitch, p.h_pitch, p.max_blob);
    float *xs = reinterpret_cast<float *>(smem + L.xs);
    __nv_bfloat16 *xp = reinterpret_cast<__nv_bfloat16 *>(smem + L.xp);
    float *ypart = reinterpret_cast<float *>(smem + L.xp);
    __nv_bfloat16 *hp = reinterpret_cast<__nv_bfloat16 *>(smem + L.hp);
    float *gu_out = reinterpret_cast<float *>(smem + L.gu);
    float *xnew = reinterpret_cast<float *>(smem + L.xnew);
    uint8_t *wbuf = smem + L.wbuf;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L.bars);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t = lane & 3;
    const int row0 = (int)(blockIdx.x / cs) * 8;                 // this cluster's block of rows
    const int D = p.d_model, OC = D / cs;                         // output columns owned by a rank
    const int U = p.d_ff / 16 / cs;                               // hidden tile rows owned by a rank
    const int RD = D / 16;
    const int xplane_w = 8 * p.x_pitch / 2, hplane_w = 8 * p.h_pitch / 2;

    auto prefetch = [&](int app, int buf) {
        // one bulk copy of this rank's blob for application `app` into weight buffer `buf`
        const int layer = p.app_layer[app];
        const int *ent = p.blob_table + ((long long)layer * cs + rank) * 2;
        const uint32_t bytes = (uint32_t)ent[1];
        const uint32_t bar = smem_u32(&bars[buf]);
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
        asm volatile(
            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
            ::"r"(smem_u32(wbuf + (size_t)buf * p.max_blob)), "l"(p.blobs + (size_t)ent[0] * 16), "r"(bytes), "r"(bar)
            : "memory");
    };

    // Both weight buffers start as zeros: a blob of zeros describes tile rows without groups, so if
    // a copy should ever fail to arrive (the bounded wait below reports it) the walk over the
    // buffer stays inside it instead of following uninitialised offsets.
    for (int i = threadIdx.x; i < 2 * p.max_blob / 16; i += kThreads)
        reinterpret_cast<uint4 *>(wbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
    __syncthreads();
    if (threadIdx.x == 0) {
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");   // zeros before the bulk copy's writes
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&bars[0])));
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(smem_u32(&bars[1])));
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        if (p.n_apps > 0) prefetch(0, 0);
    }
    // residual rows of this block -> shared memory (rows past the batch stay zero)
    for (int i = threadIdx.x; i < 8 * D / 4; i += kThreads) {
        const int r = i / (D / 4), c = (i % (D / 4)) * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (row0 + r < p.rows) v = *reinterpret_cast<const float4 *>(p.x + (long long)(row0 + r) * p.ldx + c);
        *reinterpret_cast<float4 *>(xs + r * D + c) = v;
    }
    __syncthreads();
    cluster.sync();          // every CTA of the cluster is resident before any remote access

    for (int a = 0; a < p.n_apps; ++a) {
        const int buf = a & 1;
        // ---- weights of this application (prefetched); start the next application's copy ----
        {
            const uint32_t bar = smem_u32(&bars[buf]);
            const uint32_t parity = (a >> 1) & 1;
            bool ok = false;
            for (uint32_t i = 0; i < kWaitLimit; ++i)
                if (mbar_try_wait(bar, parity)) { ok = true; break; }
            if (!ok && threadIdx.x == 0) atomicExch(p.status, 1);     // keep going: no barrier may be skipped
        }
        if (threadIdx.x == 0 && a + 1 < p.n_apps) prefetch(a + 1, buf ^ 1);
        const uint8_t *blob = wbuf + (size_t)buf * p.max_blob;
        const int *hdr = reinterpret_cast<const int *>(blob);
        const uint32_t blob_s = smem_u32(blob);
        const uint32_t gu_ptr = blob_s + hdr[2], gu_cols = blob_s + hdr[3], gu_codes = blob_s + hdr[4];
        const uint32_t dn_ptr = blob_s + hdr[5], dn_cols = blob_s + hdr[6], dn_codes = blob_s + hdr[7];
        const float scale_gu = __int_as_float(hdr[8]), scale_dn = __int_as_float(hdr[9]);
        // rmsnorm weight of this application: the copy inside the blob when the packer put one
        // there (hdr[11]), else the caller's [n_layers][d_model] array, else no normalisation
        const float *rms_w = hdr[11] ? reinterpret_cast<const float *>(blob + hdr[11])
                                     : (p.rms != nullptr ? p.rms + (size_t)p.app_layer[a] * D : nullptr);

        // ---- n = rmsnorm(x) as exact bf16 planes (warp i stages row i) ----
        {
            const int row = warp >> 1, half = warp & 1;          // two warps per row
            const float *xr = xs + row * D;
            float inv = 1.f;
            if (rms_w != nullptr) {
                float ss = 0.f;
                for (int c = lane * 4; c < D; c += 128) {
                    const float4 v = *reinterpret_cast<const float4 *>(xr + c);
                    ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                }
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                inv = 1.f / sqrtf(ss / (float)D + p.eps);
            }
            for (int c = half * 128 + lane * 4; c < D; c += 256) {
                const float4 v = *reinterpret_cast<const float4 *>(xr + c);
                float vv[4] = {v.x, v.y, v.z, v.w};
                if (rms_w != nullptr) {
                    const float4 wv = *reinterpret_cast<const float4 *>(rms_w + c);
                    vv[0] = (vv[0] * inv) * wv.x; vv[1] = (vv[1] * inv) * wv.y;
                    vv[2] = (vv[2] * inv) * wv.z; vv[3] = (vv[3] * inv) * wv.w;
                }
                for (int pl = 0; pl < P; ++pl) {
                    __nv_bfloat16 h[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        h[k] = __float2bfloat16_rn(vv[k]);
                        vv[k] -= __bfloat162float(h[k]);
                    }
                    *reinterpret_cast<uint2 *>(xp + (size_t)pl * 8 * p.x_pitch + row * p.x_pitch + c) =
                        *reinterpret_cast<uint2 *>(h);
                }
            }
        }
        __syncthreads();

        // ---- hidden slice: gate and up sums of this rank's 2U tile rows, one row per warp turn ----
        {
            uint32_t act[P];
#pragma unroll
            for (int pl = 0; pl < P; ++pl)
                act[pl] = smem_u32(xp) + (uint32_t)(pl * xplane_w + g * (p.x_pitch / 2) + t) * 4u;
            const int W = 2 * U * 16;                            // gate columns then up columns
            const int HW = U * 16;
            if (U >= kWarps) {
                // enough hidden tile rows for every warp: one warp computes the gate and the up
                // tile row of a hidden tile row and applies SwiGLU in registers
                for (int hrow = warp; hrow < U; hrow += kWarps) {
                    float ag[4] = {0.f, 0.f, 0.f, 0.f}, au[4] = {0.f, 0.f, 0.f, 0.f};
                    tile_row<P>(gu_ptr, gu_cols, gu_codes, hrow, act, lane, ag);
                    tile_row<P>(gu_ptr, gu_cols, gu_codes, U + hrow, act, lane, au);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {                // (neuron g + 8*(i>>1), row 2t + (i&1))
                        const float gv = scale_gu * ag[i], uv = scale_gu * au[i];
                        float hv = gv * (1.f / (1.f + expf(-gv))) * uv;
                        __nv_bfloat16 *o = hp + (2 * t + (i & 1)) * p.h_pitch + hrow * 16 + g + 8 * (i >> 1);
#pragma unroll
                        for (int pl = 0; pl < P; ++pl) {
                            const __nv_bfloat16 hb = __float2bfloat16_rn(hv);
                            o[(size_t)pl * 8 * p.h_pitch] = hb;
                            hv -= __bfloat162float(hb);
                        }
                    }
                }
            } else {
                for (int trow = warp; trow < 2 * U; trow += kWarps) {
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    tile_row<P>(gu_ptr, gu_cols, gu_codes, trow, act, lane, acc);
#pragma unroll
                    for (int i = 0; i < 4; ++i)                  // (neuron g + 8*(i>>1), row 2t + (i&1))
                        gu_out[(2 * t + (i & 1)) * W + trow * 16 + g + 8 * (i >> 1)] = scale_gu * acc[i];
                }
                __syncthreads();
                // silu(gate) * up -> exact bf16 planes of the hidden slice
                const int r = warp >> 1;                         // two warps per activation row
                for (int c = (warp & 1) * 32 + lane; c < HW; c += 64) {
                    const float gv = gu_out[r * W + c], uv = gu_out[r * W + HW + c];
                    float hv = gv * (1.f / (1.f + expf(-gv))) * uv;
                    __nv_bfloat16 *o = hp + r * p.h_pitch + c;
#pragma unroll
                    for (int pl = 0; pl < P; ++pl) {
                        const __nv_bfloat16 hb = __float2bfloat16_rn(hv);
                        o[(size_t)pl * 8 * p.h_pitch] = hb;
                        hv -= __bfloat162float(hb);
                    }
                }
            }
        }
        __syncthreads();

        // ---- partial down projection over this rank's hidden slice, for every output ----
        {
            uint32_t act[P];
#pragma unroll
            for (int pl = 0; pl < P; ++pl)
                act[pl] = smem_u32(hp) + (uint32_t)(pl * hplane_w + g * (p.h_pitch / 2) + t) * 4u;
            for (int trow = warp; trow < RD; trow += kWarps) {
                float acc[4] = {0.f, 0.f, 0.f, 0.f};
                tile_row<P>(dn_ptr, dn_cols, dn_codes, trow, act, lane, acc);
#pragma unroll
                for (int i = 0; i < 4; ++i)
                    ypart[(2 * t + (i & 1)) * D + trow * 16 + g + 8 * (i >> 1)] = scale_dn * acc[i];
            }
        }
        cluster.sync();      // all partial sums of the cluster are in place

        // ---- combine: this rank owns output columns [rank*OC, (rank+1)*OC) ----
        // All remote loads of an element are issued before the first add; the adds stay in
        // rank order.
        {
            float *mine = xnew + (size_t)buf * 8 * OC;
            const int r = warp >> 1;                             // two warps per activation row
            for (int cl = (warp & 1) * 32 + lane; cl < OC; cl += 64) {
                const int c = rank * OC + cl;
                float part[16];
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    if (q < 8 || cs == 16) part[q] = cluster.map_shared_rank(ypart, q)[r * D + c];
                float v = xs[r * D + c];
#pragma unroll
                for (int q = 0; q < 16; ++q)
                    if (q < 8 || cs == 16) v += part[q];                 // rank order
                mine[r * OC + cl] = v;
            }
        }
        cluster.sync();      // new residual slices published; partial sums no longer needed

        // ---- gather the new residual rows from all ranks ----
        {
            const int r = warp >> 1;                             // two warps per activation row
            const float inv_oc = 1.f / (float)OC;
#pragma unroll 3
            for (int c4 = (warp & 1) * 32 + lane; c4 < D / 4; c4 += 64) {
                const int c = c4 * 4;
                const int q = (int)(((float)c + 0.5f) * inv_oc);          // c / OC for these small integers
                const float *src = cluster.map_shared_rank(xnew, q) + (size_t)buf * 8 * OC + r * OC + (c - q * OC);
                *reinterpret_cast<float4 *>(xs + r * D + c) = *reinterpret_cast<const float4 *>(src);
            }
        }
        __syncthreads();
    }

    // this rank writes its column slice of the final rows
    for (int e = threadIdx.x; e < 8 * OC; e += kThreads) {
        const int r = e / OC, c = rank * OC + e % OC;
        if (row0 + r < p.rows) p.x[(long long)(row0 + r) * p.ldx + c] = xs[r * D + c];
    }
    cluster.sync();          // no CTA leaves while a peer may still read its shared memory
}

inline int pitch_for(int features) {
    // row pitch (bf16 elements) whose 32-bit word count is 4 mod 32: the 8 rows x 4 lanes of a
    // B-fragment load then hit 32 different banks
    const int words = features / 2;
    const int pad = ((4 - words % 32) % 32 + 32) % 32;
    return (words + pad) * 2;
}

}  // namespace

extern "C" int mortar_stack_decode(const void *blobs, const int32_t *blob_table, const int32_t *app_layer,
                                   const float *rms_weights, int32_t n_apps, int32_t n_layers,
                                   int32_t d_model, int32_t d_ff, int32_t max_blob_bytes,
                                   int32_t cluster_size, float *x, int64_t ldx, int64_t rows, float eps,
                                   int32_t n_planes, int32_t *status, void *stream) {
    if (!blobs || !blob_table || !app_layer || !x || !status) return MORTAR_ERR_NULL;
    if (n_layers <= 0) return MORTAR_ERR_SHAPE;
    if (rms_weights && (reinterpret_cast<uintptr_t>(rms_weights) % 16)) return MORTAR_ERR_ALIGN;
    if (n_apps < 0 || d_model <= 0 || d_ff <= 0 || d_model % 16 || d_ff % 16 || rows < 0 || ldx < d_model)
        return MORTAR_ERR_SHAPE;
    if (cluster_size != 8 && cluster_size != 16) return MORTAR_ERR_SHAPE;
    if ((d_ff / 16) % cluster_size || d_model % (4 * cluster_size)) return MORTAR_ERR_SHAPE;
    if (n_planes < 1 || n_planes > 3) return MORTAR_ERR_DTYPE;
    if ((reinterpret_cast<uintptr_t>(blobs) % 16) || (reinterpret_cast<uintptr_t>(x) % 16) || (ldx % 4) ||
        (max_blob_bytes % 128))
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
        v -= 1024;                                     // room for static shared variables
        void (*kernels[3])(const StackParams) = {stack_decode_kernel<1>, stack_decode_kernel<2>, stack_decode_kernel<3>};
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
    p.x = x; p.ldx = ldx; p.rows = (int)rows; p.eps = eps; p.n_planes = n_planes; p.status = status;
    p.x_pitch = pitch_for(d_model);
    p.h_pitch = pitch_for(d_ff / cluster_size);
    p.max_blob = max_blob_bytes;
    const SmemLayout L = smem_layout(d_model, d_ff, cluster_size, n_planes, p.x_pitch, p.h_pitch, max_blob_bytes);
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
    if (n_planes == 1) MORTAR_CUDA_CHECK(cudaLaunchKernelEx(&cfg, stack_decode_kernel<1>, p));
    else if (n_planes == 2) MORTAR_CUDA_CHECK(cudaLaunchKernelEx(&cfg, stack_decode_kernel<2>, p));
    else MORTAR_CUDA_CHECK(cudaLaunchKernelEx(&cfg, stack_decode_kernel<3>, p));
    return MORTAR_OK;
}
