// Harness around the REFERENCE's own masked GEMM kernel.  TEST INFRASTRUCTURE ONLY.
//
// Built by oracle/Makefile from this file plus the reference's unmodified CUTLASS headers where they
// lie in a checkout of the reference (StreamMaskedGEMM/cutlass/...); nothing of the reference is
// copied into this repository.  The harness instantiates the GEMM type the reference's driver uses
// (Volta884GemmTraits, column-major NN, 32x128x128 threadblock tile, fp16 operands and accumulators:
// StreamMaskedGEMM/perf/basic_nn.cu:250-259, :307) and calls it the way Stream_Gemm_NN does
// (basic_nn.cu:411-427): per column tile, params.initialize(M, N_cal, K_cal, alpha, A, M,
// B + off_B, K, beta, C + off_C, M, C + off_C, M) and Gemm::launch(params, mask_k, mask_n, stream)
// (cutlass/gemm/gemm.h:317-327).  Inputs come from a file instead of the driver's unseeded rand(),
// so the same seeded problem can be given to this library and the results compared.
//
// The kernel body is Volta mma.sync.m8n8k4 PTX; compiled as compute_70 PTX it is translated by the
// driver for the GPU at hand.
//
//   ref_stream_gemm <problem.bin> <result.bin>
//
// problem.bin (little endian):  int32 magic 0x54535247, M, N, K, block_num, iters;
//   int32 N_cal[block_num], K_cal[block_num], off_B[block_num], off_C[block_num];
//   per tile: int32 mask_k[K_cal[t]], int32 mask_n[128]  (relative offsets, mask_gen of basic_nn.cu:697-741);
//   fp16 A[K*M] (A^T, [K][M]);  fp16 B[N*K] (compacted tiles, column-major, ldb = K);
//   float alpha, beta;  fp16 C0[N*M] (initial C, [N][M]).
// result.bin:  fp16 C[N*M];  float microseconds per pass, timed the reference's way (one stream per
//   tile, a device synchronisation after every pass, mean of `iters` passes, basic_nn.cu:402-436).
#include <cstdio>
#include <cstdlib>
#include <vector>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include "cutlass/gemm/gemm.h"
#include "cutlass/gemm/volta884_gemm_traits.h"

typedef cutlass::gemm::Volta884GemmTraits<cutlass::MatrixLayout::kColumnMajor, cutlass::MatrixLayout::kColumnMajor,
                                          cutlass::Shape<32, 128, 128>, cutlass::Shape<32, 64, 64>, half, half, half,
                                          2>
    RefTraits;
typedef cutlass::gemm::Gemm<RefTraits> RefGemm;

#define CHECK(expr)                                                                           \
  do {                                                                                        \
    cudaError_t e_ = (expr);                                                                  \
    if (e_ != cudaSuccess) {                                                                  \
      fprintf(stderr, "%s failed: %s\n", #expr, cudaGetErrorString(e_));                      \
      return 2;                                                                               \
    }                                                                                         \
  } while (0)

template <typename T>
static bool read_vec(FILE* f, std::vector<T>* v, size_t n) {
  v->resize(n);
  return n == 0 || fread(v->data(), sizeof(T), n, f) == n;
}

int main(int argc, char** argv) {
  if (argc != 3) {
    fprintf(stderr, "usage: ref_stream_gemm <problem.bin> <result.bin>\n");
    return 1;
  }
  FILE* f = fopen(argv[1], "rb");
  if (!f) {
    fprintf(stderr, "cannot open %s\n", argv[1]);
    return 1;
  }
  int hdr[6];
  if (fread(hdr, sizeof(int), 6, f) != 6 || hdr[0] != 0x54535247) {
    fprintf(stderr, "bad problem file\n");
    return 1;
  }
  const int M = hdr[1], N = hdr[2], K = hdr[3], bn = hdr[4], iters = hdr[5];
  if (M <= 0 || N <= 0 || K <= 0 || bn <= 0 || bn > 32 || (M % 8) || (N % 8) || (K % 8)) {
    fprintf(stderr, "sizes out of range\n");
    return 1;
  }
  std::vector<int> n_cal, k_cal, off_b, off_c;
  bool ok = read_vec(f, &n_cal, bn) && read_vec(f, &k_cal, bn) && read_vec(f, &off_b, bn) && read_vec(f, &off_c, bn);
  std::vector<std::vector<int>> mk(bn), mn(bn);
  for (int t = 0; ok && t < bn; ++t) {
    // every range the kernel will touch is checked here, on the host, before anything is launched
    ok = n_cal[t] >= 0 && n_cal[t] <= 128 && k_cal[t] >= 0 && k_cal[t] <= K && off_b[t] >= 0 && off_c[t] >= 0 &&
         static_cast<long long>(off_b[t]) + static_cast<long long>(n_cal[t]) * K <= static_cast<long long>(N) * K &&
         off_c[t] % M == 0;
    ok = ok && read_vec(f, &mk[t], k_cal[t]) && read_vec(f, &mn[t], 128);
    for (int i = 0; ok && i < k_cal[t]; ++i) ok = mk[t][i] + i >= 0 && mk[t][i] + i < K;
    for (int j = 0; ok && j < n_cal[t]; ++j) ok = mn[t][j] + j >= 0 && off_c[t] / M + mn[t][j] + j < N;
  }
  std::vector<half> A, B, C0;
  float ab[2];
  ok = ok && read_vec(f, &A, static_cast<size_t>(K) * M) && read_vec(f, &B, static_cast<size_t>(N) * K) &&
       fread(ab, sizeof(float), 2, f) == 2 && read_vec(f, &C0, static_cast<size_t>(N) * M);
  fclose(f);
  if (!ok) {
    fprintf(stderr, "problem file is truncated or inconsistent\n");
    return 1;
  }

  half *dA, *dB, *dC;
  CHECK(cudaMalloc(&dA, A.size() * sizeof(half)));
  CHECK(cudaMalloc(&dB, B.size() * sizeof(half)));
  CHECK(cudaMalloc(&dC, C0.size() * sizeof(half)));
  CHECK(cudaMemcpy(dA, A.data(), A.size() * sizeof(half), cudaMemcpyHostToDevice));
  CHECK(cudaMemcpy(dB, B.data(), B.size() * sizeof(half), cudaMemcpyHostToDevice));
  std::vector<int*> dmk(bn), dmn(bn);
  for (int t = 0; t < bn; ++t) {
    CHECK(cudaMalloc(&dmk[t], (k_cal[t] > 0 ? k_cal[t] : 1) * sizeof(int)));
    CHECK(cudaMalloc(&dmn[t], 128 * sizeof(int)));
    if (k_cal[t] > 0) CHECK(cudaMemcpy(dmk[t], mk[t].data(), k_cal[t] * sizeof(int), cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(dmn[t], mn[t].data(), 128 * sizeof(int), cudaMemcpyHostToDevice));
  }
  std::vector<cudaStream_t> streams(bn);
  for (int t = 0; t < bn; ++t) CHECK(cudaStreamCreate(&streams[t]));

  const half alpha = __float2half(ab[0]), beta = __float2half(ab[1]);
  auto one_pass = [&]() -> int {
    for (int t = 0; t < bn; ++t) {
      if (n_cal[t] == 0 || k_cal[t] == 0) continue;
      RefGemm::Params params;
      int rc = params.initialize(M, n_cal[t], k_cal[t], alpha, dA, M, dB + off_b[t], K, beta, dC + off_c[t], M,
                                 dC + off_c[t], M);
      if (rc) {
        fprintf(stderr, "params.initialize failed for tile %d\n", t);
        return 3;
      }
      RefGemm::launch(params, dmk[t], dmn[t], streams[t]);
    }
    CHECK(cudaDeviceSynchronize());
    return 0;
  };

  // the result: one pass from the given initial C
  CHECK(cudaMemcpy(dC, C0.data(), C0.size() * sizeof(half), cudaMemcpyHostToDevice));
  if (int rc = one_pass()) return rc;
  CHECK(cudaGetLastError());
  std::vector<half> C(C0.size());
  CHECK(cudaMemcpy(C.data(), dC, C.size() * sizeof(half), cudaMemcpyDeviceToHost));

  // the reference's timing protocol
  float us = 0.0f;
  if (iters > 0) {
    cudaEvent_t e0, e1;
    CHECK(cudaEventCreate(&e0));
    CHECK(cudaEventCreate(&e1));
    CHECK(cudaEventRecord(e0));
    for (int i = 0; i < iters; ++i) {
      if (int rc = one_pass()) return rc;
    }
    CHECK(cudaEventRecord(e1));
    CHECK(cudaEventSynchronize(e1));
    float ms = 0.0f;
    CHECK(cudaEventElapsedTime(&ms, e0, e1));
    us = ms * 1000.0f / iters;
  }
  FILE* g = fopen(argv[2], "wb");
  if (!g || fwrite(C.data(), sizeof(half), C.size(), g) != C.size() || fwrite(&us, sizeof(float), 1, g) != 1) {
    fprintf(stderr, "cannot write %s\n", argv[2]);
    return 1;
  }
  fclose(g);
  printf("Stream  GEMM : %f us.\n", us);
  return 0;
}
