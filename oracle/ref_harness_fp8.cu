// Drives the UNMODIFIED reference kernels of cuda/gemm/fp8_gemm.cu on inputs read from a
// file and writes their raw outputs, so that the oracle can be pinned against what the
// reference itself computes.  TEST INFRASTRUCTURE ONLY.  The reference source is pulled
// in at compile time from the reference tree (-I<reference root>); nothing is copied.
//
// usage: ref_fp8 <in.bin> <out.bin> M N K G
//   in : A[M*K] f32, B[K*N] f32, sa[M*ng] f32, sb[ng*N] f32      (ng = ceil(K/G))
//   out: qA[M*K] u8, qB[K*N] u8, scaleA f32, scaleB f32, C_per_tensor[M*N] f32, C_groupwise[M*N] f32
#define main reference_main
#include "cuda/gemm/fp8_gemm.cu"
#undef main
#include <vector>

static void rd(FILE* f, void* p, size_t n) { if (fread(p, 1, n, f) != n) { fprintf(stderr, "short read\n"); exit(2); } }

int main(int argc, char** argv) {
    if (argc != 7) { fprintf(stderr, "usage\n"); return 2; }
    int M = atoi(argv[3]), N = atoi(argv[4]), K = atoi(argv[5]), G = atoi(argv[6]);
    int ng = (K + G - 1) / G;
    std::vector<float> hA((size_t)M * K), hB((size_t)K * N), hsa((size_t)M * ng), hsb((size_t)ng * N);
    FILE* f = fopen(argv[1], "rb");
    if (!f) return 2;
    rd(f, hA.data(), hA.size() * 4); rd(f, hB.data(), hB.size() * 4);
    rd(f, hsa.data(), hsa.size() * 4); rd(f, hsb.data(), hsb.size() * 4);
    fclose(f);

    float *dA, *dB, *dC, *dsc, *dsa, *dsb;
    __nv_fp8_e4m3 *qA, *qB;
    CHECK_CUDA(cudaMalloc(&dA, hA.size() * 4)); CHECK_CUDA(cudaMalloc(&dB, hB.size() * 4));
    CHECK_CUDA(cudaMalloc(&dC, (size_t)M * N * 4)); CHECK_CUDA(cudaMalloc(&dsc, 8));
    CHECK_CUDA(cudaMalloc(&dsa, hsa.size() * 4)); CHECK_CUDA(cudaMalloc(&dsb, hsb.size() * 4));
    CHECK_CUDA(cudaMalloc(&qA, hA.size())); CHECK_CUDA(cudaMalloc(&qB, hB.size()));
    CHECK_CUDA(cudaMemcpy(dA, hA.data(), hA.size() * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dB, hB.data(), hB.size() * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dsa, hsa.data(), hsa.size() * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dsb, hsb.data(), hsb.size() * 4, cudaMemcpyHostToDevice));

    quantize_to_fp8_kernel<<<1, 256>>>(dA, qA, dsc, M * K);       // launch shape of fp8_gemm.cu:181-182
    quantize_to_fp8_kernel<<<1, 256>>>(dB, qB, dsc + 1, K * N);
    float sc[2];
    CHECK_CUDA(cudaMemcpy(sc, dsc, 8, cudaMemcpyDeviceToHost));

    std::vector<uint8_t> hqA(hA.size()), hqB(hB.size());
    std::vector<float> c1((size_t)M * N), c2((size_t)M * N);
    CHECK_CUDA(cudaMemcpy(hqA.data(), qA, hqA.size(), cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(hqB.data(), qB, hqB.size(), cudaMemcpyDeviceToHost));
    fp8_gemm_per_tensor(qA, qB, dC, M, N, K, sc[0], sc[1]);
    CHECK_CUDA(cudaMemcpy(c1.data(), dC, c1.size() * 4, cudaMemcpyDeviceToHost));
    fp8_gemm_groupwise(qA, qB, dC, M, N, K, G, dsa, dsb);
    CHECK_CUDA(cudaMemcpy(c2.data(), dC, c2.size() * 4, cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaDeviceSynchronize());

    FILE* o = fopen(argv[2], "wb");
    if (!o) return 2;
    fwrite(hqA.data(), 1, hqA.size(), o); fwrite(hqB.data(), 1, hqB.size(), o);
    fwrite(sc, 4, 2, o);
    fwrite(c1.data(), 4, c1.size(), o); fwrite(c2.data(), 4, c2.size(), o);
    fclose(o);
    return 0;
}
