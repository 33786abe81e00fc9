// Dense, batched and grouped matrix products of the sequence models: C[m, n] = sum_k A[m, k] * B[n, k] with float accumulation.
//   * gemm_simt_kernel — any storage type, plain FMA (the all-32-bit mode; the tests compare the tensor-core forms with it);
//   * gemm_mma_kernel  — bf16 operands on mma.sync.m16n8k16 with a cp.async double buffer (the serving mode).
// Both take the same GemmArgs: grid.z batches with strides (per-head up-projections), or the grouped form in which every 64-row tile
// names its own weight matrix (routed experts) and A rows may be gathered through an index list.
#include "seq_kernels.cuh"
#include <stdlib.h>

namespace wf {
namespace seq {

namespace {

constexpr int BM = 64, BN = 64, BK = 16;       // kernel tile; GEMM_BM (the grouped form's row granule) is a multiple of BM

template <typename T, bool AF32, bool CF32>
__global__ void __launch_bounds__(256) gemm_simt_kernel(GemmArgs g) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tile_m = blockIdx.y, tile_n = blockIdx.x, z = blockIdx.z;
    long long grp = 0;
    if (g.tile_group) {
        const int e = g.tile_group[tile_m * BM / GEMM_BM];
        if (e < 0) return;
        grp = (long long)e * g.group_stride;
    }
    const T* B = (const T*)g.B + grp + (long long)z * g.sB;
    const char* Abase = (const char*)g.A;
    const size_t a_elt = AF32 ? 4 : sizeof(T);
    Abase += (size_t)z * g.sA * a_elt;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    // loader mapping: 64 rows x 16 k = 1024 elements, 4 per thread: row = idx / 16, k = idx % 16
    int a_src[4];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int idx = tid + q * 256;
        const int m = tile_m * BM + idx / BK;
        int r = -1;
        if (m < g.M) r = g.a_rows ? g.a_rows[m] : m;
        a_src[q] = r;
    }
    for (int k0 = 0; k0 < g.K; k0 += BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int idx = tid + q * 256;
            const int row = idx / BK, kk = idx % BK, k = k0 + kk;
            float av = 0.f;
            if (a_src[q] >= 0 && k < g.K) {
                const size_t off = (size_t)a_src[q] * g.lda + k;
                av = AF32 ? ((const float*)Abase)[off] : to_f(((const T*)Abase)[off]);
            }
            As[kk][row] = av;
            const int n = tile_n * BN + row;
            Bs[kk][row] = (n < g.N && k < g.K) ? to_f(B[(size_t)n * g.ldb + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = tile_m * BM + ty * 4 + i;
        if (m >= g.M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = tile_n * BN + tx * 4 + j;
            if (n >= g.N) continue;
            const size_t off = (size_t)z * g.sC + (size_t)m * g.ldc + n;
            if (CF32) ((float*)g.C)[off] = acc[i][j];
            else ((T*)g.C)[off] = from_f<T>(acc[i][j]);
        }
    }
}

// ---- bf16 tensor-core form: 64 x 64 x 32 tiles, 4 warps (2 x 2), each warp 32 x 32 = 2 x 4 m16n8k16 tiles -----------------------------
constexpr int MK = 32, MPAD = 8;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <bool AF32, bool CF32>
__global__ void __launch_bounds__(128) gemm_mma_kernel(GemmArgs g) {
    __shared__ __align__(16) __nv_bfloat16 As[2][BM][MK + MPAD];
    __shared__ __align__(16) __nv_bfloat16 Bs[2][BN][MK + MPAD];
    const int tile_m = blockIdx.y, tile_n = blockIdx.x, z = blockIdx.z;
    long long grp = 0;
    if (g.tile_group) {
        const int e = g.tile_group[tile_m * BM / GEMM_BM];
        if (e < 0) return;
        grp = (long long)e * g.group_stride;
    }
    const __nv_bfloat16* B = (const __nv_bfloat16*)g.B + grp + (long long)z * g.sB;
    const char* Abase = (const char*)g.A + (size_t)z * g.sA * (AF32 ? 4 : 2);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp >> 1, wn = warp & 1;
    // loader: 64 rows x 32 k = 256 chunks of 8 elements; 2 chunks per thread per operand
    int a_src[2];
#pragma unroll
    for (int q = 0; q < 2; ++q) {
        const int ch = tid + q * 128;
        const int m = tile_m * BM + ch / 4;
        a_src[q] = m < g.M ? (g.a_rows ? g.a_rows[m] : m) : -1;
    }
    const bool a_vec = !AF32 && (g.lda % 8 == 0) && (((uintptr_t)Abase & 15) == 0) && (g.K % 8 == 0);
    const bool b_vec = (g.ldb % 8 == 0) && (((uintptr_t)B & 15) == 0) && (g.K % 8 == 0);
    auto load_tile = [&](int buf, int k0) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int ch = tid + q * 128;
            const int row = ch / 4, kc = (ch % 4) * 8, k = k0 + kc;
            __nv_bfloat16* da = &As[buf][row][kc];
            if (a_vec && a_src[q] >= 0 && k + 8 <= g.K) {
                cp_async16(da, (const __nv_bfloat16*)Abase + (size_t)a_src[q] * g.lda + k);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float v = 0.f;
                    if (a_src[q] >= 0 && k + e < g.K) {
                        const size_t off = (size_t)a_src[q] * g.lda + k + e;
                        v = AF32 ? ((const float*)Abase)[off] : __bfloat162float(((const __nv_bfloat16*)Abase)[off]);
                    }
                    da[e] = __float2bfloat16_rn(v);
                }
            }
            const int n = tile_n * BN + row;
            __nv_bfloat16* db = &Bs[buf][row][kc];
            if (b_vec && n < g.N && k + 8 <= g.K) {
                cp_async16(db, B + (size_t)n * g.ldb + k);
            } else {
#pragma unroll
                for (int e = 0; e < 8; ++e) db[e] = (n < g.N && k + e < g.K) ? B[(size_t)n * g.ldb + k + e] : __float2bfloat16_rn(0.f);
            }
        }
        cp_async_commit();
    };
    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
    const int nk = (g.K + MK - 1) / MK;
    load_tile(0, 0);
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) { load_tile(buf ^ 1, (kt + 1) * MK); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < MK; ks += 16) {
            uint32_t a[2][4], b[4][2];
            const int r = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int m0 = wm * 32 + i * 16;
                a[i][0] = *(const uint32_t*)&As[buf][m0 + r][ks + c];
                a[i][1] = *(const uint32_t*)&As[buf][m0 + r + 8][ks + c];
                a[i][2] = *(const uint32_t*)&As[buf][m0 + r][ks + c + 8];
                a[i][3] = *(const uint32_t*)&As[buf][m0 + r + 8][ks + c + 8];
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n0 = wn * 32 + j * 8;
                b[j][0] = *(const uint32_t*)&Bs[buf][n0 + r][ks + c];
                b[j][1] = *(const uint32_t*)&Bs[buf][n0 + r][ks + c + 8];
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], a[i], b[j]);
        }
        __syncthreads();
    }
    const int r = lane >> 2, c = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = tile_m * BM + wm * 32 + i * 16 + r + h * 8;
                if (m >= g.M) continue;
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int n = tile_n * BN + wn * 32 + j * 8 + c + e;
                    if (n >= g.N) continue;
                    const size_t off = (size_t)z * g.sC + (size_t)m * g.ldc + n;
                    const float v = acc[i][j][h * 2 + e];
                    if (CF32) ((float*)g.C)[off] = v;
                    else ((__nv_bfloat16*)g.C)[off] = __float2bfloat16_rn(v);
                }
            }
}

// ---- few-row form (decoding): the weight matrix is streamed once, 16 bytes per lane per load; a warp owns GV_RPW output columns and
// all MR <= 8 activation rows, which every warp re-reads through L1.  With `pair_expert` set, grid.y walks (token, expert) pairs instead:
// pair p multiplies ONE activation row (p / pair_div) with the weight matrix of expert pair_expert[p] (routed experts while decoding).
constexpr int GV_WARPS = 8, GV_RPW = 2;

template <typename T> struct Vec16;
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };
template <> struct Vec16<float> { static constexpr int N = 4; };

template <typename T>
__device__ __forceinline__ void load_vec(const T* p, float (&out)[Vec16<T>::N]);
template <>
__device__ __forceinline__ void load_vec<__nv_bfloat16>(const __nv_bfloat16* p, float (&out)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { out[2 * i] = __uint_as_float(w[i] << 16); out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}
template <>
__device__ __forceinline__ void load_vec<float>(const float* p, float (&out)[4]) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}

struct PairArgs { const int32_t* pair_expert; int n_experts; int pair_div; };

template <typename T, int MR, bool AF32, bool CF32>
__global__ void __launch_bounds__(GV_WARPS * 32) gemv_rows_kernel(GemmArgs g, PairArgs pa) {
    constexpr int VN = Vec16<T>::N;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const T* B = (const T*)g.B;
    int a_row0 = 0, c_row0 = 0, rows = g.M;
    if (pa.pair_expert) {
        const int pr = blockIdx.y;
        const int e = pa.pair_expert[pr];
        if (e < 0 || e >= pa.n_experts) return;
        B += (long long)e * g.group_stride;
        a_row0 = pr / pa.pair_div; c_row0 = pr; rows = 1;
    }
    const int n0 = (blockIdx.x * GV_WARPS + warp) * GV_RPW;
    if (n0 >= g.N) return;
    float acc[GV_RPW][MR];
#pragma unroll
    for (int r = 0; r < GV_RPW; ++r)
#pragma unroll
        for (int m = 0; m < MR; ++m) acc[r][m] = 0.f;
    const int kvec = g.K / VN;                       // the launcher guarantees K % VN == 0 and 16-byte aligned rows
    for (int kv = lane; kv < kvec; kv += 32) {
        const int k = kv * VN;
        float b[GV_RPW][VN];
#pragma unroll
        for (int r = 0; r < GV_RPW; ++r) {
            const int n = n0 + r < g.N ? n0 + r : g.N - 1;
            load_vec<T>(B + (size_t)n * g.ldb + k, b[r]);
        }
#pragma unroll
        for (int m = 0; m < MR; ++m) {
            if (m < rows) {
                float a[VN];
                if (AF32) {
#pragma unroll
                    for (int i = 0; i < VN; ++i) a[i] = ((const float*)g.A)[(size_t)(a_row0 + m) * g.lda + k + i];
                } else {
                    load_vec<T>((const T*)g.A + (size_t)(a_row0 + m) * g.lda + k, a);
                }
#pragma unroll
                for (int r = 0; r < GV_RPW; ++r)
#pragma unroll
                    for (int i = 0; i < VN; ++i) acc[r][m] = fmaf(a[i], b[r][i], acc[r][m]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < GV_RPW; ++r)
#pragma unroll
        for (int m = 0; m < MR; ++m) {
            float v = acc[r][m];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m < rows && n0 + r < g.N) {
                const size_t off = (size_t)(c_row0 + m) * g.ldc + n0 + r;
                if (CF32) ((float*)g.C)[off] = v; else ((T*)g.C)[off] = from_f<T>(v);
            }
        }
}

template <typename T, int MR>
void gemv_dispatch(const GemmArgs& g, const PairArgs& pa, dim3 grid, cudaStream_t s) {
    if (g.a_f32) { if (g.c_f32) gemv_rows_kernel<T, MR, true, true><<<grid, GV_WARPS * 32, 0, s>>>(g, pa); else gemv_rows_kernel<T, MR, true, false><<<grid, GV_WARPS * 32, 0, s>>>(g, pa); }
    else { if (g.c_f32) gemv_rows_kernel<T, MR, false, true><<<grid, GV_WARPS * 32, 0, s>>>(g, pa); else gemv_rows_kernel<T, MR, false, false><<<grid, GV_WARPS * 32, 0, s>>>(g, pa); }
}

template <typename T>
bool gemv_ok(const GemmArgs& g) {
    constexpr int VN = Vec16<T>::N;
    const size_t ea = g.a_f32 ? 4 : sizeof(T);
    return g.K % VN == 0 && g.ldb % VN == 0 && (((uintptr_t)g.B) & 15) == 0 && (g.lda * ea) % 16 == 0 && (((uintptr_t)g.A) & 15) == 0 &&
           (g.group_stride * (long long)sizeof(T)) % 16 == 0;
}

template <typename T>
void gemv_launch(const GemmArgs& g, const PairArgs& pa, int rows, int ny, cudaStream_t s) {
    dim3 grid((g.N + GV_WARPS * GV_RPW - 1) / (GV_WARPS * GV_RPW), ny);
    if (rows <= 1) gemv_dispatch<T, 1>(g, pa, grid, s);
    else if (rows <= 2) gemv_dispatch<T, 2>(g, pa, grid, s);
    else if (rows <= 4) gemv_dispatch<T, 4>(g, pa, grid, s);
    else gemv_dispatch<T, 8>(g, pa, grid, s);
}

template <typename T>
void simt_dispatch(const GemmArgs& g, dim3 grid, cudaStream_t s) {
    if (g.a_f32) { if (g.c_f32) gemm_simt_kernel<T, true, true><<<grid, 256, 0, s>>>(g); else gemm_simt_kernel<T, true, false><<<grid, 256, 0, s>>>(g); }
    else { if (g.c_f32) gemm_simt_kernel<T, false, true><<<grid, 256, 0, s>>>(g); else gemm_simt_kernel<T, false, false><<<grid, 256, 0, s>>>(g); }
}

int g_force_simt = -1, g_tc_min = -1;

}  // namespace

int launch_gemm(int dt, const GemmArgs& g, cudaStream_t s) {
    if (g.M <= 0 || g.N <= 0 || g.batch <= 0) return WF_OK;
    if (g.K <= 0 || !g.A || !g.B || !g.C) { set_error("gemm: bad arguments (M %d N %d K %d)", g.M, g.N, g.K); return WF_ERR_INVALID; }
    if (g_tc_min < 0) { const char* e = getenv("WF_SEQ_TC_MIN"); g_tc_min = e ? atoi(e) : 17; }
    if (g_force_simt < 0) { const char* e = getenv("WF_SEQ_GEMM_SIMT"); g_force_simt = (e && atoi(e)) ? 1 : 0; }
    const bool few = g.batch == 1 && !g.tile_group && !g.a_rows && g.M <= 8;
    if ((g.algo == 0 && few) || g.algo == 4) {      // decoding: stream the weights once
        const PairArgs none{nullptr, 0, 1};
        if (few && dt == WF_F32 && gemv_ok<float>(g)) { gemv_launch<float>(g, none, g.M, 1, s); return launch_check(cudaGetLastError(), "gemv_rows"); }
        if (few && dt == WF_BF16 && gemv_ok<__nv_bfloat16>(g)) { gemv_launch<__nv_bfloat16>(g, none, g.M, 1, s); return launch_check(cudaGetLastError(), "gemv_rows"); }
        if (g.algo == 4) { set_error("gemm: the few-row form does not take this shape"); return WF_ERR_UNSUPPORTED; }
    }
    dim3 grid((g.N + BN - 1) / BN, (g.M + BM - 1) / BM, g.batch);
    if (grid.y > 65535u || grid.z > 65535u) { set_error("gemm: grid too large"); return WF_ERR_UNSUPPORTED; }
    if (g.algo == 3 && (dt != WF_BF16 || !gemm_tc_usable(g))) { set_error("gemm: the tcgen05 form does not take this shape"); return WF_ERR_UNSUPPORTED; }
    if (dt == WF_F32) simt_dispatch<float>(g, grid, s);
    else if (g.algo == 1 || (g.algo == 0 && g_force_simt)) simt_dispatch<__nv_bfloat16>(g, grid, s);
    else if (g.algo == 3 || (g.algo == 0 && g.M >= g_tc_min && gemm_tc_usable(g))) return launch_gemm_tc(g, g.n_groups, s);
    else {
        if (g.a_f32) { if (g.c_f32) gemm_mma_kernel<true, true><<<grid, 128, 0, s>>>(g); else gemm_mma_kernel<true, false><<<grid, 128, 0, s>>>(g); }
        else { if (g.c_f32) gemm_mma_kernel<false, true><<<grid, 128, 0, s>>>(g); else gemm_mma_kernel<false, false><<<grid, 128, 0, s>>>(g); }
    }
    return launch_check(cudaGetLastError(), "gemm");
}

bool gemv_pairs_usable(int dt, const GemmArgs& g) {
    return dt == WF_F32 ? gemv_ok<float>(g) : gemv_ok<__nv_bfloat16>(g);
}

int launch_gemv_pairs(int dt, const GemmArgs& g, const int32_t* pair_expert, int n_experts, int pairs, int pair_div, cudaStream_t s) {
    if (pairs <= 0 || g.N <= 0) return WF_OK;
    if (pairs > 65535 || !gemv_pairs_usable(dt, g)) { set_error("gemv_pairs: unsupported shape"); return WF_ERR_UNSUPPORTED; }
    const PairArgs pa{pair_expert, n_experts, pair_div};
    if (dt == WF_F32) gemv_launch<float>(g, pa, 1, pairs, s); else gemv_launch<__nv_bfloat16>(g, pa, 1, pairs, s);
    return launch_check(cudaGetLastError(), "gemv_pairs");
}

}  // namespace seq
}  // namespace wf
