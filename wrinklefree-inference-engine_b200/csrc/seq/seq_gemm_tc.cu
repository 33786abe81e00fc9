// bf16 matrix product on the 5th-generation tensor cores for prompt-sized row counts:  C[m, n] = sum_k A[m, k] * B[n, k], fp32 accumulate.
//
// Persistent CTA per SM, 6 warps: 4 epilogue (one per TMEM lane quarter), 1 TMA producer, 1 MMA issuer — the pipeline of the LM head kernel
// (lm_head_tc.cu) turned into a general linear layer:
//   * a tile is 128 weight rows (UMMA M, TMEM lanes) x 128 tokens (UMMA N, TMEM columns); a stage is 64 k of both (16 KB + 16 KB) brought by
//     cp.async.bulk.tensor.2d with the 128-byte swizzle the UMMA descriptors expect; rows past the tensor and k past K are zero-filled by
//     the TMA unit, so no shape needs padding; 6 stages = 192 KB;
//   * accumulators are double-buffered in TMEM (2 x 128 columns): the epilogue of tile i overlaps the stream of tile i + 1;
//   * one thread chosen by elect.sync issues 4 x tcgen05.mma (M128 N128 K16) per stage and commits the stage back to the producer;
//   * epilogue: tcgen05.ld 32x32b.x32 -> a thread holds its weight row's values for 32 tokens; a warp's store of one token covers 32
//     consecutive n (one 128-byte line of float, or 64 bytes of bf16);
//   * consecutive tiles of a CTA wave share the token tile and walk the weight rows, so activations are re-read from L2, weights streamed;
//   * grouped form (routed experts): every 128-token tile names its expert; the weight tensor map covers all experts' rows stacked.
// Every wait is bounded: a wait that runs out records an error word the host checks, and the CTA drains and leaves.
#include "seq_kernels.cuh"
#include <cuda.h>

namespace wf {
namespace seq {

namespace {

constexpr int TC_ROWS = 128;                       // weight rows per tile (UMMA M)
constexpr int TC_TOK = 128;                        // tokens per tile (UMMA N)
constexpr int TC_KC = 64;                          // k per stage: 128 bytes of bf16 = one swizzle atom row
constexpr int TC_STAGES = 6;
constexpr int TC_W_BYTES = TC_ROWS * 128;          // 16 KB
constexpr int TC_A_BYTES = TC_TOK * 128;           // 16 KB
constexpr int TC_STAGE_BYTES = TC_W_BYTES + TC_A_BYTES;
constexpr int TC_SMEM = TC_STAGES * TC_STAGE_BYTES + 1024;
constexpr int TC_THREADS = 6 * 32;
constexpr int TC_TMEM_COLS = 256;
constexpr uint32_t TC_SPIN_LIMIT = 1u << 24;

struct TcParams {
    int M, N, K;
    int n_tiles, tiles;
    void* C; int ldc, c_f32;
    const int32_t* tile_group;     // per 128-token tile: expert, or < 0 = skip (null: dense)
    int group_w_rows;              // weight rows between consecutive experts in the stacked tensor
    int* err;
};

__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {   // K-major tile, 128-byte rows, 8-row groups 1024 B apart
    uint64_t d = 0;
    d |= (uint64_t)((saddr & 0x3ffffu) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}
// D f32, A bf16 (K-major), B bf16 (K-major), N, M
constexpr uint32_t make_idesc(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// bounded wait on an mbarrier phase; false when it ran out
__device__ __forceinline__ bool wait_bounded(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < TC_SPIN_LIMIT; ++i) {
        uint32_t ok;
        asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}
#define TC_LD32(taddr, v)                                                                                              \
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"       \
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"                            \
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),      \
                   "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), \
                   "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]),           \
                   "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),           \
                   "=r"(v[30]), "=r"(v[31])                                                                             \
                 : "r"(taddr) : "memory")

__global__ void __launch_bounds__(TC_THREADS, 1) gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                                                                const TcParams p) {
    extern __shared__ unsigned char smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[TC_STAGES], empty_bar[TC_STAGES], tfull_bar[2], tempty_bar[2];
    __shared__ uint32_t tmem_base_s;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t ring = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const int my_tiles = p.tiles > (int)blockIdx.x ? (p.tiles - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x : 0;
    const int kchunks = (p.K + TC_KC - 1) / TC_KC;

    if (tid == 0) {
        for (int s = 0; s < TC_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&tfull_bar[b], 1); mbar_init(&tempty_bar[b], 4); }
        fence_mbar_init();
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "n"(TC_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_base_s;

    // every role walks the same list of tiles and skips the same ones; `it` counts ring items, `done` counts tiles that were computed
    if (warp == 4) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_w) : "memory");
            asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
            int it = 0;
            bool ok = true;
            for (int tl = 0; tl < my_tiles && ok; ++tl) {
                const int tile = blockIdx.x + tl * gridDim.x;
                const int mt = tile / p.n_tiles, nt = tile - mt * p.n_tiles;
                int w_row = nt * TC_ROWS;
                if (p.tile_group) {
                    const int e = p.tile_group[mt];
                    if (e < 0) continue;
                    w_row += e * p.group_w_rows;
                }
                for (int kc = 0; kc < kchunks; ++kc, ++it) {
                    const int s = it % TC_STAGES;
                    if (it >= TC_STAGES && !wait_bounded(smem_u32(&empty_bar[s]), (uint32_t)(((it / TC_STAGES) & 1) ^ 1))) { ok = false; break; }
                    mbar_expect_tx(&full_bar[s], TC_STAGE_BYTES);
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(ring + s * TC_STAGE_BYTES), "l"(&tmap_w), "r"(kc * TC_KC), "r"(w_row), "r"(smem_u32(&full_bar[s])) : "memory");
                    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                                 ::"r"(ring + s * TC_STAGE_BYTES + TC_W_BYTES), "l"(&tmap_a), "r"(kc * TC_KC), "r"(mt * TC_TOK), "r"(smem_u32(&full_bar[s])) : "memory");
                }
            }
            if (!ok) atomicExch(p.err, 1);
        }
    } else if (warp == 5) {
        // ------------------------------------------------------------ MMA issuer: one elected thread runs the whole loop
        constexpr uint32_t idesc = make_idesc(TC_ROWS, TC_TOK);
        const uint64_t adesc0 = smem_desc_sw128(ring);
        const uint64_t bdesc0 = smem_desc_sw128(ring + TC_W_BYTES);
        uint32_t elected;
        asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(elected));
        if (elected) {
            int it = 0, done = 0;
            bool ok = true;
            for (int tl = 0; tl < my_tiles && ok; ++tl) {
                const int tile = blockIdx.x + tl * gridDim.x;
                const int mt = tile / p.n_tiles;
                if (p.tile_group && p.tile_group[mt] < 0) continue;
                const int buf = done & 1;
                if (done >= 2 && !wait_bounded(smem_u32(&tempty_bar[buf]), (uint32_t)(((done >> 1) & 1) ^ 1))) { ok = false; break; }
                const uint32_t d_tmem = tmem + buf * TC_TOK;
                for (int kc = 0; kc < kchunks; ++kc, ++it) {
                    const int s = it % TC_STAGES;
                    if (!wait_bounded(smem_u32(&full_bar[s]), (uint32_t)((it / TC_STAGES) & 1))) { ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t ad = adesc0 + (uint64_t)(s * (TC_STAGE_BYTES >> 4));
                    const uint64_t bd = bdesc0 + (uint64_t)(s * (TC_STAGE_BYTES >> 4));
                    mma_bf16_ss(d_tmem, ad, bd, idesc, kc != 0 ? 1u : 0u);          // 16 k per instruction = 32 bytes = +2 in the descriptor
                    mma_bf16_ss(d_tmem, ad + 2, bd + 2, idesc, 1u);
                    mma_bf16_ss(d_tmem, ad + 4, bd + 4, idesc, 1u);
                    mma_bf16_ss(d_tmem, ad + 6, bd + 6, idesc, 1u);
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&empty_bar[s])) : "memory");
                }
                if (!ok) break;
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(&tfull_bar[buf])) : "memory");
                ++done;
            }
            if (!ok) atomicExch(p.err, 2);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue warps: TMEM -> C
        const int q = warp;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        int done = 0;
        bool ok = true;
        for (int tl = 0; tl < my_tiles && ok; ++tl) {
            const int tile = blockIdx.x + tl * gridDim.x;
            const int mt = tile / p.n_tiles, nt = tile - mt * p.n_tiles;
            if (p.tile_group && p.tile_group[mt] < 0) continue;
            const int buf = done & 1;
            const int n = nt * TC_ROWS + q * 32 + lane;                    // this thread's weight row = output column
            const bool n_ok = n < p.N;
            if (!wait_bounded(smem_u32(&tfull_bar[buf]), (uint32_t)((done >> 1) & 1))) { ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c = 0; c < TC_TOK / 32; ++c) {
                uint32_t r[32];
                TC_LD32(tmem + lane_base + buf * TC_TOK + c * 32, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (c == TC_TOK / 32 - 1) {
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&tempty_bar[buf]);
                }
                const int m0 = mt * TC_TOK + c * 32;
                const int mcnt = p.M - m0 < 32 ? p.M - m0 : 32;            // warp-uniform
                if (n_ok) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        if (j < mcnt) {
                            const size_t off = (size_t)(m0 + j) * p.ldc + n;
                            if (p.c_f32) ((float*)p.C)[off] = __uint_as_float(r[j]);
                            else ((__nv_bfloat16*)p.C)[off] = __float2bfloat16_rn(__uint_as_float(r[j]));
                        }
                    }
                }
            }
            ++done;
        }
        if (!ok && lane == 0) atomicExch(p.err, 3);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 5) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "n"(TC_TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
DevOnce g_attr;
int* g_err_dev[64] = {nullptr};

int encode_2d(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t cols, uint64_t row_stride_elems, uint32_t box_rows) {
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)row_stride_elems * 2};
    const cuuint32_t box[2] = {TC_KC, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = g_encode(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)base, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                 CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) { set_error("gemm_tc: tensor map failed (%d)", (int)cr); return WF_ERR_CUDA; }
    return WF_OK;
}

}  // namespace

bool gemm_tc_usable(const GemmArgs& g) {
    if (g.a_f32 || g.batch != 1 || g.a_rows) return false;
    if (g.lda % 8 || g.ldb % 8 || ((uintptr_t)g.A & 15) || ((uintptr_t)g.B & 15) || g.K < 8 || g.lda < g.K || g.ldb < g.K) return false;
    if (g.tile_group && (g.group_stride % g.ldb)) return false;
    return true;
}

int gemm_tc_error(cudaStream_t s) {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev > 63 || !g_err_dev[dev]) return 0;
    int h = 0;
    if (cudaMemcpyAsync(&h, g_err_dev[dev], 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
    if (cudaStreamSynchronize(s) != cudaSuccess) return -1;
    return h;
}

// n_groups: number of stacked weight matrices (1 when dense)
int launch_gemm_tc(const GemmArgs& g, int n_groups, cudaStream_t s) {
    if (g_attr.need()) cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM);
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult qr;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qr) == cudaSuccess && qr == cudaDriverEntryPointSuccess)
            g_encode = (EncodeTiledFn)fn;
    }
    if (!g_encode) { set_error("gemm_tc: cuTensorMapEncodeTiled unavailable"); return WF_ERR_CUDA; }
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev > 63) dev = 0;
    if (!g_err_dev[dev]) {
        if (cuda_check(cudaMalloc((void**)&g_err_dev[dev], 4), "cudaMalloc")) return WF_ERR_CUDA;
        if (cuda_check(cudaMemset(g_err_dev[dev], 0, 4), "memset")) return WF_ERR_CUDA;
    }
    CUtensorMap tw, ta;
    const int group_w_rows = g.tile_group ? (int)(g.group_stride / g.ldb) : 0;
    const uint64_t w_rows = g.tile_group ? (uint64_t)(n_groups - 1) * group_w_rows + g.N : (uint64_t)g.N;
    if (int rc = encode_2d(&tw, g.B, w_rows, g.K, g.ldb, TC_ROWS)) return rc;
    if (int rc = encode_2d(&ta, g.A, g.M, g.K, g.lda, TC_TOK)) return rc;
    TcParams p;
    p.M = g.M; p.N = g.N; p.K = g.K;
    p.n_tiles = (g.N + TC_ROWS - 1) / TC_ROWS;
    p.tiles = p.n_tiles * ((g.M + TC_TOK - 1) / TC_TOK);
    p.C = g.C; p.ldc = g.ldc; p.c_f32 = g.c_f32;
    p.tile_group = g.tile_group; p.group_w_rows = group_w_rows;
    p.err = g_err_dev[dev];
    const int sms = sm_count();
    gemm_tc_kernel<<<p.tiles < sms ? p.tiles : sms, TC_THREADS, TC_SMEM, s>>>(tw, ta, p);
    return launch_check(cudaGetLastError(), "gemm_tc");
}

}  // namespace seq
}  // namespace wf
