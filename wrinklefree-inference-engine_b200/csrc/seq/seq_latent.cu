// Latent attention over a paged cache of (latent c_j, shared rotated key part kr_j) rows, with a sliding window.
// Per head the key is k_j = [W_uk c_j, kr_j] and the value W_uv c_j; neither is ever materialised: the query's unrotated part is carried
// through the key up-projection once (qa = W_uk^T q, a per-head batched product done by the caller), scores are qa . c_j + qr . kr_j, the
// weighted sum runs over the latents and the value up-projection is applied to that sum (again a batched product).  Scores, softmax and
// the weighted sum are float.
#include "seq_kernels.cuh"
#include <math.h>

namespace wf {
namespace seq {

namespace {

// pair (i, i + dims / 2) of a vector at position pos: angle pos * base^(-2 i / dims), all in float
__device__ __forceinline__ void rope_pair(float u, float v, int i, int dims, float base, int pos, float* ou, float* ov) {
    const float f = powf(base, -2.0f * (float)i / (float)dims);
    const float a = (float)pos * f;
    float sn, cs;
    sincosf(a, &sn, &cs);
    *ou = u * cs - v * sn;
    *ov = v * cs + u * sn;
}

template <typename T>
__global__ void latent_q_prep_kernel(Batch b, LatentDims L, const float* __restrict__ q, int ldq, T* __restrict__ qn, float* __restrict__ qr) {
    const int i = blockIdx.x;
    const int pos = b.tok_pos[i];
    const int per = L.d + L.r, half = L.rope_dims / 2;
    for (int idx = blockIdx.y * blockDim.x + threadIdx.x; idx < L.H * per; idx += gridDim.y * blockDim.x) {
        const int h = idx / per, c = idx % per;
        const float* src = q + (size_t)i * ldq + (size_t)h * per;
        if (c < L.d) { qn[((size_t)i * L.H + h) * L.d + c] = from_f<T>(src[c]); continue; }
        const int e = c - L.d;
        float* dst = qr + ((size_t)i * L.H + h) * L.r;
        if (e < half) {
            float ou, ov;
            rope_pair(src[L.d + e], src[L.d + e + half], e, L.rope_dims, L.rope_base, pos, &ou, &ov);
            dst[e] = ou; dst[e + half] = ov;
        } else if (e >= L.rope_dims) {
            dst[e] = src[c];
        }
    }
}

// one block per token: latent RMS norm + rotary of the shared key part, stored as T in the token's cache row
template <typename T>
__global__ void latent_kv_write_kernel(Batch b, LatentDims L, const float* __restrict__ dkv, int ld, const T* __restrict__ w, float eps, PagedCache pc) {
    __shared__ float scratch[33];
    const int i = blockIdx.x;
    const int sq = b.tok_seq[i], pos = b.tok_pos[i];
    const int page = pc.block_table[(size_t)b.seq_slot[sq] * pc.max_blocks + pos / pc.page_size];
    T* row = (T*)pc.pool + (size_t)page * pc.page_stride + pc.layer_off + (size_t)(pos % pc.page_size) * (L.R + L.r);
    const float* src = dkv + (size_t)i * ld;
    float ss = 0.f;
    for (int c = threadIdx.x; c < L.R; c += blockDim.x) ss += src[c] * src[c];
    ss = block_sum(ss, scratch);
    const float inv = 1.f / sqrtf(ss / (float)L.R + eps);
    for (int c = threadIdx.x; c < L.R; c += blockDim.x) row[c] = from_f<T>(src[c] * inv * to_f(w[c]));
    const int half = L.rope_dims / 2;
    for (int e = threadIdx.x; e < L.r; e += blockDim.x) {
        if (e < half) {
            float ou, ov;
            rope_pair(src[L.R + e], src[L.R + e + half], e, L.rope_dims, L.rope_base, pos, &ou, &ov);
            row[L.R + e] = from_f<T>(ou); row[L.R + e + half] = from_f<T>(ov);
        } else if (e >= L.rope_dims) {
            row[L.R + e] = from_f<T>(src[L.R + e]);
        }
    }
}

constexpr int LA_WARPS = 4;
constexpr int LA_MAXR = 16;    // latent size up to 32 * 16
constexpr int LA_MAXr = 8;     // rotated size up to 32 * 8

// One block per (token, head).  Its warps take the visible positions round-robin; a warp handles one position at a time with its lanes
// over the dimensions (coalesced reads of the cache row), keeps a running max / sum / weighted latent sum, and the warps' partial results
// are merged through shared memory at the end.
template <typename T>
__global__ void __launch_bounds__(LA_WARPS * 32) latent_attn_kernel(Batch b, LatentDims L, const float* __restrict__ qa, const float* __restrict__ qr,
                                                                      PagedCache pc, T* __restrict__ out) {
    extern __shared__ float sm[];   // [LA_WARPS][R] partial sums, then [LA_WARPS] m, [LA_WARPS] l
    const int i = blockIdx.x, h = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int sq = b.tok_seq[i], pos = b.tok_pos[i];
    const int lo = pos - L.window + 1 > 0 ? pos - L.window + 1 : 0;
    const int32_t* bt = pc.block_table + (size_t)b.seq_slot[sq] * pc.max_blocks;
    const int width = L.R + L.r;
    const float* qa_h = qa + ((size_t)i * L.H + h) * L.R;
    const float* qr_h = qr + ((size_t)i * L.H + h) * L.r;
    float qreg[LA_MAXR], rreg[LA_MAXr], acc[LA_MAXR];
#pragma unroll
    for (int t = 0; t < LA_MAXR; ++t) { const int c = lane + 32 * t; qreg[t] = c < L.R ? qa_h[c] : 0.f; acc[t] = 0.f; }
#pragma unroll
    for (int t = 0; t < LA_MAXr; ++t) { const int c = lane + 32 * t; rreg[t] = c < L.r ? qr_h[c] : 0.f; }
    float m = -INFINITY, l = 0.f;
    for (int j = lo + warp; j <= pos; j += LA_WARPS) {
        const int page = bt[j / pc.page_size];
        const T* row = (const T*)pc.pool + (size_t)page * pc.page_stride + pc.layer_off + (size_t)(j % pc.page_size) * width;
        float cv[LA_MAXR];
        float part = 0.f;
#pragma unroll
        for (int t = 0; t < LA_MAXR; ++t) {
            const int c = lane + 32 * t;
            cv[t] = c < L.R ? to_f(row[c]) : 0.f;
            part = fmaf(qreg[t], cv[t], part);
        }
#pragma unroll
        for (int t = 0; t < LA_MAXr; ++t) {
            const int c = lane + 32 * t;
            if (c < L.r) part = fmaf(rreg[t], to_f(row[L.R + c]), part);
        }
        const float sc = warp_sum(part) * L.scale;
        const float mn = fmaxf(m, sc);
        const float corr = expf(m - mn);      // m = -inf on the first position: exp(-inf) = 0
        const float p = expf(sc - mn);
        l = l * corr + p;
#pragma unroll
        for (int t = 0; t < LA_MAXR; ++t) acc[t] = fmaf(p, cv[t], acc[t] * corr);
        m = mn;
    }
    float* part_sum = sm;
    float* part_m = sm + LA_WARPS * L.R;
    float* part_l = part_m + LA_WARPS;
#pragma unroll
    for (int t = 0; t < LA_MAXR; ++t) { const int c = lane + 32 * t; if (c < L.R) part_sum[warp * L.R + c] = acc[t]; }
    if (lane == 0) { part_m[warp] = m; part_l[warp] = l; }
    __syncthreads();
    float mg = -INFINITY;
#pragma unroll
    for (int w = 0; w < LA_WARPS; ++w) mg = fmaxf(mg, part_m[w]);
    float lg = 0.f, sc_w[LA_WARPS];
#pragma unroll
    for (int w = 0; w < LA_WARPS; ++w) { sc_w[w] = part_m[w] == -INFINITY ? 0.f : expf(part_m[w] - mg); lg += part_l[w] * sc_w[w]; }
    const float inv = 1.f / lg;
    for (int c = threadIdx.x; c < L.R; c += blockDim.x) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < LA_WARPS; ++w) v += part_sum[w * L.R + c] * sc_w[w];
        out[((size_t)i * L.H + h) * L.R + c] = from_f<T>(v * inv);
    }
}

int check_dims(const LatentDims& L) {
    if (L.R > 32 * LA_MAXR || L.r > 32 * LA_MAXr) { set_error("latent attention: kv_rank %d / rot_dim %d above the supported %d / %d", L.R, L.r, 32 * LA_MAXR, 32 * LA_MAXr); return WF_ERR_UNSUPPORTED; }
    if (L.rope_dims > L.r || (L.rope_dims & 1) || L.window < 1) { set_error("latent attention: rotary dims %d of %d, window %d", L.rope_dims, L.r, L.window); return WF_ERR_INVALID; }
    return WF_OK;
}

}  // namespace

int launch_latent_q_prep(int dt, const Batch& b, const LatentDims& L, const float* q, int ldq, void* qn, float* qr, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (int rc = check_dims(L)) return rc;
    const dim3 grid(b.n, b.n < 64 ? (L.H * (L.d + L.r) + 255) / 256 : 1);
    if (dt == WF_BF16) latent_q_prep_kernel<<<grid, 256, 0, s>>>(b, L, q, ldq, (__nv_bfloat16*)qn, qr);
    else latent_q_prep_kernel<<<grid, 256, 0, s>>>(b, L, q, ldq, (float*)qn, qr);
    return launch_check(cudaGetLastError(), "latent_q_prep");
}

int launch_latent_kv_write(int dt, const Batch& b, const LatentDims& L, const float* dkv, int ld, const void* w, float eps, const PagedCache& pc,
                           cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (int rc = check_dims(L)) return rc;
    if (dt == WF_BF16) latent_kv_write_kernel<<<b.n, 128, 0, s>>>(b, L, dkv, ld, (const __nv_bfloat16*)w, eps, pc);
    else latent_kv_write_kernel<<<b.n, 128, 0, s>>>(b, L, dkv, ld, (const float*)w, eps, pc);
    return launch_check(cudaGetLastError(), "latent_kv_write");
}

int launch_latent_attn(int dt, const Batch& b, const LatentDims& L, const float* qa, const float* qr, const PagedCache& pc, void* out, cudaStream_t s) {
    if (b.n <= 0) return WF_OK;
    if (int rc = check_dims(L)) return rc;
    if (L.H > 65535) { set_error("latent attention: too many heads"); return WF_ERR_UNSUPPORTED; }
    dim3 grid(b.n, L.H);
    const size_t smem = ((size_t)LA_WARPS * L.R + 2 * LA_WARPS) * sizeof(float);
    if (dt == WF_BF16) latent_attn_kernel<<<grid, LA_WARPS * 32, smem, s>>>(b, L, qa, qr, pc, (__nv_bfloat16*)out);
    else latent_attn_kernel<<<grid, LA_WARPS * 32, smem, s>>>(b, L, qa, qr, pc, (float*)out);
    return launch_check(cudaGetLastError(), "latent_attn");
}

}  // namespace seq
}  // namespace wf
