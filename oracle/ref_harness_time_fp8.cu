// Times the UNMODIFIED reference FP8 GEMM kernels of cuda/gemm/fp8_gemm.cu on a GPU, for context beside the CPU arm of
// the benchmark: what the reference's own CUDA code does on the same part.  TEST / MEASUREMENT INFRASTRUCTURE ONLY.  The
// reference source is pulled in at compile time from the reference tree (-I<reference root>); nothing is copied.
//
// usage: ref_time_fp8 M N K G [iters]
//   operands are arbitrary valid E4M3 bytes and unit scales (the kernels' time does not depend on the values)
//   prints one line: "groupwise_ms <t> per_tensor_ms <t>"  (mean over iters, CUDA events, after one warm-up launch each)
#define main reference_main
#include "cuda/gemm/fp8_gemm.cu"
#undef main
#include <vector>

int main(int argc, char** argv) {
    if (argc < 5) { fprintf(stderr, "usage: ref_time_fp8 M N K G [iters]\n"); return 2; }
    const int M = atoi(argv[1]), N = atoi(argv[2]), K = atoi(argv[3]), G = atoi(argv[4]);
    const int iters = argc > 5 ? atoi(argv[5]) : 1;
    if (M <= 0 || N <= 0 || K <= 0 || G <= 0 || iters <= 0) return 2;
    const int ng = (K + G - 1) / G;
    __nv_fp8_e4m3 *A, *B;
    float *C, *sa, *sb;
    CHECK_CUDA(cudaMalloc(&A, (size_t)M * K));
    CHECK_CUDA(cudaMalloc(&B, (size_t)K * N));
    CHECK_CUDA(cudaMalloc(&C, (size_t)M * N * 4));
    CHECK_CUDA(cudaMalloc(&sa, (size_t)M * ng * 4));
    CHECK_CUDA(cudaMalloc(&sb, (size_t)ng * N * 4));
    CHECK_CUDA(cudaMemset(A, 0x38, (size_t)M * K));      // 0x38 = 1.0 in E4M3
    CHECK_CUDA(cudaMemset(B, 0x38, (size_t)K * N));
    std::vector<float> ones((size_t)(M > N ? M : N) * ng, 1.0f);
    CHECK_CUDA(cudaMemcpy(sa, ones.data(), (size_t)M * ng * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(sb, ones.data(), (size_t)ng * N * 4, cudaMemcpyHostToDevice));
    cudaEvent_t e0, e1;
    CHECK_CUDA(cudaEventCreate(&e0));
    CHECK_CUDA(cudaEventCreate(&e1));
    float gw = 0.f, pt = 0.f;
    fp8_gemm_groupwise(A, B, C, M, N, K, G, sa, sb);
    CHECK_CUDA(cudaEventRecord(e0));
    for (int i = 0; i < iters; ++i) fp8_gemm_groupwise(A, B, C, M, N, K, G, sa, sb);
    CHECK_CUDA(cudaEventRecord(e1));
    CHECK_CUDA(cudaEventSynchronize(e1));
    CHECK_CUDA(cudaEventElapsedTime(&gw, e0, e1));
    fp8_gemm_per_tensor(A, B, C, M, N, K, 1.0f, 1.0f);
    CHECK_CUDA(cudaEventRecord(e0));
    for (int i = 0; i < iters; ++i) fp8_gemm_per_tensor(A, B, C, M, N, K, 1.0f, 1.0f);
    CHECK_CUDA(cudaEventRecord(e1));
    CHECK_CUDA(cudaEventSynchronize(e1));
    CHECK_CUDA(cudaEventElapsedTime(&pt, e0, e1));
    printf("groupwise_ms %.4f per_tensor_ms %.4f\n", gw / iters, pt / iters);
    return 0;
}
