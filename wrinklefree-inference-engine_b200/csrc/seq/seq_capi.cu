// Per-op C entry points of the sequence-model kernels (tests and measurements call the launchers the engine uses).
#include "seq_kernels.cuh"
#include "wf_seq.h"

using namespace wf;
using namespace wf::seq;

extern "C" int wf_seq_op_gemm(int dtype, const void* A, int a_f32, int lda, const void* B, int ldb, void* C, int c_f32, int ldc, int M, int N, int K,
                              const int32_t* tile_group, long long group_stride, int n_groups, int algo, void* stream) {
    GemmArgs g;
    g.A = A; g.a_f32 = a_f32; g.lda = lda; g.B = B; g.ldb = ldb; g.C = C; g.c_f32 = c_f32; g.ldc = ldc; g.M = M; g.N = N; g.K = K;
    g.tile_group = tile_group; g.group_stride = group_stride; g.n_groups = n_groups; g.algo = algo;
    const int rc = launch_gemm(dtype == WF_SEQ_F32 ? WF_F32 : WF_BF16, g, (cudaStream_t)stream);
    if (rc) return rc;
    if (algo == 3 || algo == 0) {
        if (cuda_check(cudaStreamSynchronize((cudaStream_t)stream), "wf_seq_op_gemm")) return WF_ERR_CUDA;
        if (dtype != WF_SEQ_F32 && gemm_tc_error((cudaStream_t)stream)) { set_error("wf_seq_op_gemm: a bounded wait of the tcgen05 kernel ran out"); return WF_ERR_CUDA; }
    }
    return WF_OK;
}
