// Drives the UNMODIFIED reference kernels of cuda/gemm/grouped_gemm.cu (fixed and variable
// grouped GEMM) on inputs read from a file and writes their raw outputs.
// TEST INFRASTRUCTURE ONLY; the reference source is pulled in at compile time.
//
// usage: ref_grouped <in.bin> <out.bin> G M N K  m_0 ... m_{G-1}
//   in : A[G*M*K] f32, B[G*K*N] f32
//   out: C_fixed[G*M*N] f32, C_variable[sum(m_g)*N] f32
// The variable run uses group g's first m_g rows of A (A_offset = g*M*K elements) and packs
// the outputs back to back.
#define main reference_main
#include "cuda/gemm/grouped_gemm.cu"
#undef main
#include <vector>

static void rd(FILE* f, void* p, size_t n) { if (fread(p, 1, n, f) != n) { fprintf(stderr, "short read\n"); exit(2); } }

int main(int argc, char** argv) {
    if (argc < 7) { fprintf(stderr, "usage\n"); return 2; }
    int G = atoi(argv[3]), M = atoi(argv[4]), N = atoi(argv[5]), K = atoi(argv[6]);
    if (argc != 7 + G) { fprintf(stderr, "need %d row counts\n", G); return 2; }
    size_t na = (size_t)G * M * K, nb = (size_t)G * K * N, nc = (size_t)G * M * N;
    std::vector<float> hA(na), hB(nb), c1(nc);
    FILE* f = fopen(argv[1], "rb");
    if (!f) return 2;
    rd(f, hA.data(), na * 4); rd(f, hB.data(), nb * 4);
    fclose(f);
    std::vector<GemmProblem> probs(G);
    int total = 0, max_m = 0;
    for (int g = 0; g < G; g++) {
        int mg = atoi(argv[7 + g]);
        probs[g] = GemmProblem{mg, N, K, g * M * K, g * K * N, total * N};
        total += mg;
        if (mg > max_m) max_m = mg;
    }
    float *dA, *dB, *dC;
    GemmProblem* dP;
    CHECK_CUDA(cudaMalloc(&dA, na * 4)); CHECK_CUDA(cudaMalloc(&dB, nb * 4)); CHECK_CUDA(cudaMalloc(&dC, nc * 4));
    CHECK_CUDA(cudaMalloc(&dP, sizeof(GemmProblem) * G));
    CHECK_CUDA(cudaMemcpy(dA, hA.data(), na * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dB, hB.data(), nb * 4, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dP, probs.data(), sizeof(GemmProblem) * G, cudaMemcpyHostToDevice));
    grouped_gemm_fixed(dA, dB, dC, M, N, K, G);
    CHECK_CUDA(cudaMemcpy(c1.data(), dC, nc * 4, cudaMemcpyDeviceToHost));
    std::vector<float> c2((size_t)total * N);
    CHECK_CUDA(cudaMemset(dC, 0, nc * 4));
    if (max_m > 0) grouped_gemm_variable(dA, dB, dC, dP, G, max_m, N);
    CHECK_CUDA(cudaMemcpy(c2.data(), dC, c2.size() * 4, cudaMemcpyDeviceToHost));
    FILE* o = fopen(argv[2], "wb");
    if (!o) return 2;
    fwrite(c1.data(), 4, c1.size(), o); fwrite(c2.data(), 4, c2.size(), o);
    fclose(o);
    return 0;
}
