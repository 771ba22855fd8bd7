// ReMoE tile router in two launches: the query projection (a dense fp32 product, many CTAs) and
// everything after it (one CTA per row).  Same arithmetic as TileRouter.forward
// (morph/model/routing.py:159-284): q = LayerNorm(x Wq^T + iter_embed); product-key scores
// sa = q[:d/2] Ka^T, sb = q[d/2:] Kb^T; group logits from the nsk x nsk sums sa[a] + sb[b];
// gate = relu(logit - k-th largest) * k / max(sum, 1e-6).  The decode engine of the reference
// does the same in two Triton launches for ONE row and the 1:1 product map only
// (morph/kernels/triton/fused_router.py:101-139); here any number of rows and all three maps.
#include <cuda_runtime.h>
#include <cstdint>
#include <mutex>
#include "common.h"

namespace {

constexpr int kProjRows = 8;        // activation rows a warp accumulates for one output at a time
constexpr int kTailThreads = 256;

// qv[b, o] = sum_i x[b, i] * wq[o, i] + iter_vec[o].  One warp per output feature, kProjRows rows
// of x per pass (blockIdx.y), so a weight row is read once per 8 rows.  VEC: 128-bit loads (d a
// multiple of 4, rows and weights 16-byte aligned).
template <bool VEC>
__global__ void __launch_bounds__(256)
router_project_kernel(const float *x, long long ldx, long long rows, int d, const float *wq,
                      const float *iter_vec, float *qv) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int o = blockIdx.x * 8 + warp;
    if (o >= d) return;
    const long long b0 = (long long)blockIdx.y * kProjRows;
    float acc[kProjRows];
#pragma unroll
    for (int r = 0; r < kProjRows; ++r) acc[r] = 0.f;
    const float *w = wq + (long long)o * d;
    const float *xr[kProjRows];
#pragma unroll
    for (int r = 0; r < kProjRows; ++r)
        xr[r] = x + (b0 + r < rows ? b0 + r : rows - 1) * ldx;       // clamped rows are discarded
    if (VEC) {
        for (int i = lane * 4; i < d; i += 128) {
            const float4 wv = __ldg(reinterpret_cast<const float4 *>(w + i));
#pragma unroll
            for (int r = 0; r < kProjRows; ++r) {
                const float4 xv = __ldg(reinterpret_cast<const float4 *>(xr[r] + i));
                acc[r] = fmaf(xv.x, wv.x, acc[r]); acc[r] = fmaf(xv.y, wv.y, acc[r]);
                acc[r] = fmaf(xv.z, wv.z, acc[r]); acc[r] = fmaf(xv.w, wv.w, acc[r]);
            }
        }
    } else {
        for (int i = lane; i < d; i += 32) {
            const float wv = __ldg(w + i);
#pragma unroll
            for (int r = 0; r < kProjRows; ++r) acc[r] = fmaf(__ldg(xr[r] + i), wv, acc[r]);
        }
    }
#pragma unroll
    for (int r = 0; r < kProjRows; ++r)
        for (int off = 16; off > 0; off >>= 1) acc[r] += __shfl_xor_sync(0xffffffffu, acc[r], off);
    if (lane == 0) {
        const float bias = iter_vec ? iter_vec[o] : 0.f;
#pragma unroll
        for (int r = 0; r < kProjRows; ++r)
            if (b0 + r < rows) qv[(b0 + r) * d + o] = acc[r] + bias;
    }
}

__device__ __forceinline__ float block_sum(float v, float *scratch) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                                   // scratch may still be read from the last call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = 0.f;
    for (int w = 0; w < kTailThreads / 32; ++w) t += scratch[w];
    return t;
}

// One CTA per row.  Dynamic shared memory: q[d] | prod[nsk*nsk] | logits[G] | sa[nsk] | sb[nsk].
__global__ void __launch_bounds__(kTailThreads)
router_tail_kernel(const float *qv, int d, const float *ln_w, const float *ln_b, float ln_eps,
                   const float *ska, const float *skb, int nsk, const float *gbias, int G, int k,
                   float *gates, long long ld_gates) {
    extern __shared__ float sm[];
    __shared__ float scratch[kTailThreads / 32];
    __shared__ float kth_s;
    float *q = sm, *prod = q + d, *logits = prod + nsk * nsk, *sa = logits + G, *sb = sa + nsk;
    const long long row = blockIdx.x;
    const float *qr = qv + row * d;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int d2 = d / 2, np = nsk * nsk;

    // LayerNorm over d (biased variance, as torch.nn.LayerNorm)
    float s = 0.f;
    for (int i = tid; i < d; i += kTailThreads) { const float v = qr[i]; q[i] = v; s += v; }
    const float mean = block_sum(s, scratch) / (float)d;
    float s2 = 0.f;
    for (int i = tid; i < d; i += kTailThreads) { const float c = q[i] - mean; s2 += c * c; }
    const float rstd = 1.f / sqrtf(block_sum(s2, scratch) / (float)d + ln_eps);
    for (int i = tid; i < d; i += kTailThreads) q[i] = (q[i] - mean) * rstd * ln_w[i] + ln_b[i];
    __syncthreads();

    // sub-key scores: 2*nsk dot products of length d/2, one warp each
    for (int j = warp; j < 2 * nsk; j += kTailThreads / 32) {
        const bool second = j >= nsk;
        const float *key = (second ? skb : ska) + (long long)(second ? j - nsk : j) * d2;
        const float *qh = q + (second ? d2 : 0);
        float a = 0.f;
        for (int i = lane; i < d2; i += 32) a = fmaf(qh[i], __ldg(key + i), a);
        for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
        if (lane == 0) (second ? sb : sa)[second ? j - nsk : j] = a;
    }
    __syncthreads();
    for (int pidx = tid; pidx < np; pidx += kTailThreads) prod[pidx] = sa[pidx / nsk] + sb[pidx % nsk];
    __syncthreads();

    // group logits: 1:1 map, the G largest products in descending order, or products repeated
    if (np == G) {
        for (int g = tid; g < G; g += kTailThreads) logits[g] = prod[g] + gbias[g];
    } else if (np > G) {
        for (int pidx = tid; pidx < np; pidx += kTailThreads) {
            const float v = prod[pidx];
            int rank = 0;                                // position in a stable descending sort
            for (int j = 0; j < np; ++j) rank += (prod[j] > v) || (prod[j] == v && j < pidx);
            if (rank < G) logits[rank] = v + gbias[rank];
        }
    } else {
        for (int g = tid; g < G; g += kTailThreads) logits[g] = prod[g % np] + gbias[g];
    }
    __syncthreads();

    // k-th largest value by exact descending rank (ties by index, the order torch.topk yields)
    if (tid == 0) kth_s = 0.f;
    __syncthreads();
    if (k < G) {
        for (int g = tid; g < G; g += kTailThreads) {
            const float v = logits[g];
            int rank = 0;
            for (int j = 0; j < G; ++j) rank += (logits[j] > v) || (logits[j] == v && j < g);
            if (rank == k - 1) kth_s = v;
        }
        __syncthreads();
    }
    const float kth = k < G ? kth_s : 0.f;
    float gs = 0.f;
    for (int g = tid; g < G; g += kTailThreads) {
        const float v = fmaxf(logits[g] - kth, 0.f);
        logits[g] = v;
        gs += v;
    }
    const float total = fmaxf(block_sum(gs, scratch), 1e-6f);
    const float mul = (float)k / total;
    for (int g = tid; g < G; g += kTailThreads) gates[row * ld_gates + g] = logits[g] * mul;
}

// The same for token blocks: 8 rows per CTA, one warp per row for everything but the sub-key
// scores, where a warp takes a key and all 8 rows, so the 2*nsk keys (d/2 floats each) are read
// once per 8 rows instead of once per row.  Dynamic shared memory:
// q[8][d] | prod[8][nsk*nsk] | logits[8][G] | sa[8][nsk] | sb[8][nsk] | sort keys[8][n_sort] (64-bit).
// The "G largest products in descending order" map and the k-th largest logit come from a warp's
// bitonic sort of its row (the one-row kernel counts ranks instead: fine for a handful of rows,
// quadratic work for a token block).
constexpr int kTailRows = 8;

__device__ __forceinline__ float warp_sum(float v) {
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
    return v;
}

// A float as an unsigned integer of the same order; with the element's index in the low word
// (inverted) a descending sort of the 64-bit keys is the stable descending sort of the values.
__device__ __forceinline__ unsigned long long sort_key(float v, int idx) {
    uint32_t u = __float_as_uint(v);
    u = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
    return ((unsigned long long)u << 32) | (unsigned long long)(0xffffffffu - (uint32_t)idx);
}

// Bitonic sort of n (a power of two) keys in shared memory by one warp, descending.
__device__ __forceinline__ void warp_sort_desc(unsigned long long *keys, int n, int lane) {
    for (int k = 2; k <= n; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int t = lane; t < n / 2; t += 32) {
                // the t-th pair of this stage: i has bit j clear, its partner has it set
                const int i = ((t & ~(j - 1)) << 1) | (t & (j - 1)), l = i | j;
                const unsigned long long a = keys[i], b = keys[l];
                const bool descending = (i & k) == 0;
                if (descending ? a < b : a > b) { keys[i] = b; keys[l] = a; }
            }
            __syncwarp();
        }
    }
}

__global__ void __launch_bounds__(kTailThreads)
router_tail_rows_kernel(const float *qv, long long rows, int d, const float *ln_w, const float *ln_b, float ln_eps,
                        const float *ska, const float *skb, int nsk, const float *gbias, int G, int k,
                        int n_sort, float *gates, long long ld_gates) {
    extern __shared__ __align__(16) float sm[];
    const int np = nsk * nsk, d2 = d / 2;
    float *q = sm, *prod = q + kTailRows * d, *logits = prod + kTailRows * np, *sa = logits + kTailRows * G;
    float *sb = sa + kTailRows * nsk;
    // 8-byte aligned start of the sort keys
    unsigned long long *keys_all = reinterpret_cast<unsigned long long *>(
        sm + ((kTailRows * (d + np + G + 2 * nsk) + 1) & ~1));
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long row0 = (long long)blockIdx.x * kTailRows;

    {   // LayerNorm of row `warp` (biased variance, as torch.nn.LayerNorm); rows past the end are zeros
        const long long row = row0 + warp;
        float *qr = q + warp * d;
        if (row < rows) {
            const float *src = qv + row * d;
            float s = 0.f;
            for (int i = lane; i < d; i += 32) { const float v = src[i]; qr[i] = v; s += v; }
            const float mean = warp_sum(s) / (float)d;
            float s2 = 0.f;
            for (int i = lane; i < d; i += 32) { const float c = qr[i] - mean; s2 += c * c; }
            const float rstd = 1.f / sqrtf(warp_sum(s2) / (float)d + ln_eps);
            for (int i = lane; i < d; i += 32) qr[i] = (qr[i] - mean) * rstd * ln_w[i] + ln_b[i];
        } else {
            for (int i = lane; i < d; i += 32) qr[i] = 0.f;
        }
    }
    __syncthreads();

    // sub-key scores: warp j takes key j against all 8 rows
    for (int j = warp; j < 2 * nsk; j += kTailThreads / 32) {
        const bool second = j >= nsk;
        const float *key = (second ? skb : ska) + (long long)(second ? j - nsk : j) * d2;
        const float *qh = q + (second ? d2 : 0);
        float a[kTailRows];
#pragma unroll
        for (int r = 0; r < kTailRows; ++r) a[r] = 0.f;
        for (int i = lane; i < d2; i += 32) {
            const float kv = __ldg(key + i);
#pragma unroll
            for (int r = 0; r < kTailRows; ++r) a[r] = fmaf(qh[r * d + i], kv, a[r]);
        }
#pragma unroll
        for (int r = 0; r < kTailRows; ++r) {
            const float t = warp_sum(a[r]);
            if (lane == 0) (second ? sb : sa)[r * nsk + (second ? j - nsk : j)] = t;
        }
    }
    __syncthreads();

    // from here on warp w finishes row w by itself
    const long long row = row0 + warp;
    if (row >= rows) return;
    float *pr = prod + warp * np, *lg = logits + warp * G;
    const float *sar = sa + warp * nsk, *sbr = sb + warp * nsk;
    unsigned long long *keys = keys_all + (size_t)warp * n_sort;
    for (int pidx = lane; pidx < np; pidx += 32) pr[pidx] = sar[pidx / nsk] + sbr[pidx % nsk];
    __syncwarp();
    if (np == G) {
        for (int g = lane; g < G; g += 32) lg[g] = pr[g] + gbias[g];
    } else if (np > G) {
        // stable descending sort of the products; the first G, in that order, are the logits
        for (int i = lane; i < n_sort; i += 32) keys[i] = i < np ? sort_key(pr[i], i) : 0ull;
        __syncwarp();
        warp_sort_desc(keys, n_sort, lane);
        for (int g = lane; g < G; g += 32) lg[g] = pr[0xffffffffu - (uint32_t)keys[g]] + gbias[g];
    } else {
        for (int g = lane; g < G; g += 32) lg[g] = pr[g % np] + gbias[g];
    }
    __syncwarp();
    float kth = 0.f;
    if (k < G) {
        // k-th largest logit: position k-1 of the sorted logits
        for (int i = lane; i < n_sort; i += 32) keys[i] = i < G ? sort_key(lg[i], i) : 0ull;
        __syncwarp();
        warp_sort_desc(keys, n_sort, lane);
        kth = lg[0xffffffffu - (uint32_t)keys[k - 1]];
    }
    float gs = 0.f;
    for (int g = lane; g < G; g += 32) {
        const float v = fmaxf(lg[g] - kth, 0.f);
        lg[g] = v;
        gs += v;
    }
    const float mul = (float)k / fmaxf(warp_sum(gs), 1e-6f);
    __syncwarp();
    for (int g = lane; g < G; g += 32) gates[row * ld_gates + g] = lg[g] * mul;
}

}  // namespace

extern "C" int mortar_router_gates(const float *x, int64_t ldx, int64_t rows, int32_t d_model,
                                   const float *wq, const float *iter_vec, const float *ln_weight,
                                   const float *ln_bias, float ln_eps, const float *sub_keys_a,
                                   const float *sub_keys_b, int32_t n_sub_keys, const float *group_bias,
                                   int32_t n_groups, int32_t k, float *qv_scratch, float *gates,
                                   int64_t ld_gates, void *stream) {
    // wq == NULL: qv_scratch already holds the projected query (x wq^T + iter_vec), e.g. from a
    // library GEMM at prefill scale; only the second launch runs
    if ((wq && !x) || !ln_weight || !ln_bias || !sub_keys_a || !sub_keys_b || !group_bias || !qv_scratch || !gates)
        return MORTAR_ERR_NULL;
    if (rows < 0 || d_model <= 0 || (d_model & 1) || (wq && ldx < d_model) || n_sub_keys <= 0 || n_groups <= 0 ||
        k <= 0 || ld_gates < n_groups)
        return MORTAR_ERR_SHAPE;
    if (rows == 0) return MORTAR_OK;
    if (rows > 0x7fffffffLL || (rows + kProjRows - 1) / kProjRows > 65535) return MORTAR_ERR_CAPACITY;
    const size_t smem = sizeof(float) * ((size_t)d_model + (size_t)n_sub_keys * n_sub_keys + n_groups + 2 * (size_t)n_sub_keys);
    if (smem > 200 * 1024) return MORTAR_ERR_CAPACITY;
    cudaStream_t st = (cudaStream_t)stream;
    dim3 grid((d_model + 7) / 8, (unsigned)((rows + kProjRows - 1) / kProjRows));
    const bool vec = (d_model % 4) == 0 && (ldx % 4) == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0 &&
                     (reinterpret_cast<uintptr_t>(wq) % 16) == 0;
    if (wq) {
        if (vec) router_project_kernel<true><<<grid, 256, 0, st>>>(x, ldx, rows, d_model, wq, iter_vec, qv_scratch);
        else router_project_kernel<false><<<grid, 256, 0, st>>>(x, ldx, rows, d_model, wq, iter_vec, qv_scratch);
        MORTAR_CUDA_CHECK(cudaGetLastError());
    }
    // token blocks: 8 rows per CTA (the sub keys are read once per 8 rows); fewer rows: one CTA per row
    int n_sort = 2;                                           // keys per row: a power of two >= max(products, groups)
    while (n_sort < n_sub_keys * n_sub_keys || n_sort < n_groups) n_sort <<= 1;
    const size_t smem8 = sizeof(float) * ((size_t)kTailRows * ((size_t)d_model + (size_t)n_sub_keys * n_sub_keys + n_groups +
                                                                2 * (size_t)n_sub_keys) + 2) +
                         sizeof(unsigned long long) * (size_t)kTailRows * n_sort;
    {   // both tail kernels may use up to 200 KB of dynamic shared memory: opt in once per device
        static bool opted[64] = {false};
        static std::mutex m;
        int dev = 0;
        MORTAR_CUDA_CHECK(cudaGetDevice(&dev));
        if (dev < 0 || dev >= 64) return MORTAR_ERR_CAPACITY;
        std::lock_guard<std::mutex> lock(m);
        if (!opted[dev]) {
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(router_tail_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            MORTAR_CUDA_CHECK(cudaFuncSetAttribute(router_tail_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            opted[dev] = true;
        }
    }
    if (rows >= 64 && smem8 <= 200 * 1024) {
        router_tail_rows_kernel<<<(unsigned)((rows + kTailRows - 1) / kTailRows), kTailThreads, smem8, st>>>(
            qv_scratch, rows, d_model, ln_weight, ln_bias, ln_eps, sub_keys_a, sub_keys_b, n_sub_keys, group_bias,
            n_groups, k, n_sort, gates, ld_gates);
        MORTAR_CUDA_CHECK(cudaGetLastError());
        return MORTAR_OK;
    }
    router_tail_kernel<<<(unsigned)rows, kTailThreads, smem, st>>>(qv_scratch, d_model, ln_weight, ln_bias, ln_eps,
                                                                    sub_keys_a, sub_keys_b, n_sub_keys, group_bias,
                                                                    n_groups, k, gates, ld_gates);
    MORTAR_CUDA_CHECK(cudaGetLastError());
    return MORTAR_OK;
}
