// Drives the UNMODIFIED reference kernels of cuda/gemm/fp4_gemm.cu on inputs read from a
// file and writes their raw outputs.  TEST INFRASTRUCTURE ONLY; the reference source is
// pulled in at compile time from the reference tree (-I<reference root>).
//
// usage: ref_fp4 <in.bin> <out.bin> M N K        (K % 32 == 0, K*N % 32 == 0)
//   in : A[M*K] f32, B[K*N] f32
//   out: pA[M*K/2] u8, sA[M*K/32] f32, pB[K*N/2] u8, sB[K*N/32] f32, C_nvfp4[M*N] f32, C_mxfp4[M*N] f32
// As in the reference's own driver (fp4_gemm.cu:184-190) both operands are quantised over
// their FLAT buffers and B's scales are then consumed as [K/32, N].
#define main reference_main
#include "cuda/gemm/fp4_gemm.cu"
#undef main
#include <vector>

static void rd(FILE* f, void* p, size_t n) { if (fread(p, 1, n, f) != n) { fprintf(stderr, "short read\n"); exit(2); } }

int main(int argc, char** argv) {
    if (argc != 6) { fprintf(stderr, "usage\n"); return 2; }
    int M = atoi(argv[3]), N = atoi(argv[4]), K = atoi(argv[5]);
    size_t na = (size_t)M * K, nb = (size_t)K * N;
    std::vector<float> hA(na), hB(nb);
    FILE* f = fopen(argv[1], "rb");
    if (!f) return 2;
    rd(f, hA.data(), na * 4); rd(f, hB.data(), nb * 4);
    fclose(f);

    float *dA, *dB, *dC, *dSA, *dSB;
    packed_fp4_t *pA, *pB;
    int nba = (int)((na + 31) / 32), nbb = (int)((nb + 31) / 32);
    CHECK_CUDA(cudaMalloc(&dA, na * 4)); CHECK_CUDA(cudaMalloc(&dB, nb * 4));
    CHECK_CUDA(cudaMalloc(&pA, (na + 1) / 2)); CHECK_CUDA(cudaMalloc(&pB, (nb + 1) / 2));
    CHECK_CUDA(cudaMalloc(&dSA, (size_t)nba * 4)); CHECK_CUDA(cudaMalloc(&dSB, (size_t)nbb * 4));
    CHECK_CUDA(cudaMalloc(&dC, (size_t)M * N * 4));
    CHECK_CUDA(cudaMemcpy(dA, hA.data(), na * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dB, hB.data(), nb * 4, cudaMemcpyHostToDevice));
    quantize_fp32_to_nvfp4<<<(nba + 255) / 256, 256>>>(dA, pA, dSA, (int)na);
    quantize_fp32_to_nvfp4<<<(nbb + 255) / 256, 256>>>(dB, pB, dSB, (int)nb);
    CHECK_CUDA(cudaDeviceSynchronize());

    std::vector<uint8_t> hpA((na + 1) / 2), hpB((nb + 1) / 2);
    std::vector<float> hsA(nba), hsB(nbb), c1((size_t)M * N), c2((size_t)M * N);
    CHECK_CUDA(cudaMemcpy(hpA.data(), pA, hpA.size(), cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(hpB.data(), pB, hpB.size(), cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(hsA.data(), dSA, hsA.size() * 4, cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(hsB.data(), dSB, hsB.size() * 4, cudaMemcpyDeviceToHost));
    fp4_gemm(pA, pB, dC, dSA, dSB, M, N, K, false);
    CHECK_CUDA(cudaMemcpy(c1.data(), dC, c1.size() * 4, cudaMemcpyDeviceToHost));
    fp4_gemm(pA, pB, dC, dSA, dSB, M, N, K, true);
    CHECK_CUDA(cudaMemcpy(c2.data(), dC, c2.size() * 4, cudaMemcpyDeviceToHost));

    FILE* o = fopen(argv[2], "wb");
    if (!o) return 2;
    fwrite(hpA.data(), 1, hpA.size(), o); fwrite(hsA.data(), 4, hsA.size(), o);
    fwrite(hpB.data(), 1, hpB.size(), o); fwrite(hsB.data(), 4, hsB.size(), o);
    fwrite(c1.data(), 4, c1.size(), o); fwrite(c2.data(), 4, c2.size(), o);
    fclose(o);
    return 0;
}
