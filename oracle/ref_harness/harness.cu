// Harness around the UNMODIFIED reference sources (included from where they lie; nothing is copied):
// builds the reference's Bert_Model<__half> (cuBLAS GEMMs, its own CUDA kernels, ncclAllReduce),
// fills every weight / bias / LayerNorm parameter / mask / input from the seeded generator of
// include/liger_rng.h (the reference leaves them uninitialised), replays the function-assembled
// kernel vector the way its Scheduler::run_sequential does (src/schedule.h:204-219: every closure
// in order on one stream), times it with CUDA events and, on request, dumps the output.
//
// TEST / BASELINE INFRASTRUCTURE: built into oracle/_ref/ by oracle/ref_harness/Makefile; none of this
// repository's kernels are linked into it.
//
//   liger_ref_harness <batch> <seq> <head_num> <size_per_head> <layers> <steps> <warmup> [dump_file]
//
// Rank / world size come from the MPI stand-in's environment (RANK / WORLD_SIZE under torchrun).
// The reference's workspace slot for the attention scores is max_batch*max_seq*H/ws elements although
// the scores need batch*heads/ws*seq^2 (src/layer/bert_layer.h:111-112): with seq > size_per_head the
// scores overflow into the next slot and the PV GEMM reads what it is overwriting.  The model is
// therefore constructed with max_seq_len = max(seq, ceil(seq^2 / size_per_head)) and run at `seq`.
// Everything the reference headers include is included first, so that the `class -> struct` switch
// below touches only the reference's own class definitions: Bert_Encoder keeps its sub-layers in
// the default-private part of a `class` (src/layer/bert.h:18-35) and the harness must reach the
// weights they own.  The reference sources themselves are not modified.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cuda_runtime_api.h>
#include <cublas_v2.h>
#include <math.h>
#include <mpi.h>
#include <nccl.h>
#include <sys/select.h>
#include <sys/time.h>
#include <unistd.h>

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <fstream>
#include <functional>
#include <iomanip>
#include <iostream>
#include <nlohmann/json.hpp>
#include <ostream>
#include <sstream>
#include <string>
#include <type_traits>
#include <unordered_map>
#include <vector>

#define class struct
#include "src/communicator.h"
#include "src/init.h"
#include "src/layer/bert.h"
#undef class

#include "liger_rng.h"

enum { W_Q = 0, W_K = 1, W_V = 2, W_O = 3, W_UP = 4, W_DOWN = 5, B_Q = 6, B_K = 7, B_V = 8, B_UP = 9,
       LN1_G = 10, LN1_B = 11, LN2_G = 12, LN2_B = 13 };

__global__ void fill_window(__half* dst, int rows, int cols, int row0, int col0, int ld, uint32_t seed, uint32_t id,
                            float mean, float std) {
  const size_t total = (size_t)rows * cols;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / cols), c = (int)(i % cols);
    reinterpret_cast<uint16_t*>(dst)[i] =
        lg_normal_half_bits(seed, id, (uint64_t)(row0 + r) * (uint64_t)ld + (uint64_t)(col0 + c), mean, std);
  }
}
__global__ void fill_const(__half* dst, size_t n, float v) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    dst[i] = __float2half(v);
}
static void fw(__half* dst, int rows, int cols, int row0, int col0, int ld, uint32_t id, float mean, float std) {
  fill_window<<<1184, 256>>>(dst, rows, cols, row0, col0, ld, 0u, id, mean, std);
}

int main(int argc, char* argv[]) {
  if (argc < 8) {
    fprintf(stderr, "usage: %s batch seq head_num size_per_head layers steps warmup [dump_file]\n", argv[0]);
    return 2;
  }
  int batch = atoi(argv[1]), seq = atoi(argv[2]), head_num = atoi(argv[3]), size_per_head = atoi(argv[4]);
  int layers = atoi(argv[5]), steps = atoi(argv[6]), warmup = atoi(argv[7]);
  const char* dump = argc > 8 ? argv[8] : nullptr;
  int world_size, world_rank;
  ncclComm_t ncclcomm = createNcclComm(argc, argv, world_size, world_rank);

  int max_seq = seq;
  const int need = (seq * seq + size_per_head - 1) / size_per_head;
  if (need > max_seq) max_seq = need;
  int kernel_num = world_size == 1 ? 14 : 16, factor = 8, rq_interval = 1000;
  StaticNvInitParam SParams(world_rank, world_size, ncclcomm, 1);
  BertInitParam BertParams(batch, max_seq, head_num, size_per_head, layers, kernel_num, factor, rq_interval);

  // buffers exactly as test_no_schedule allocates them (src/test_schedule.h:55-66)
  const int k = size_per_head * head_num, n = k;
  const size_t m = (size_t)max_seq * batch;
  __half *input, *output, *workspace;
  if (cudaMalloc((void**)&input, sizeof(__half) * m * k) != cudaSuccess ||
      cudaMalloc((void**)&output, sizeof(__half) * m * k) != cudaSuccess ||
      cudaMalloc((void**)&workspace, sizeof(__half) * m * n * 80) != cudaSuccess) {
    fprintf(stderr, "rank %d: cudaMalloc of the reference's buffers failed (workspace %.1f GB)\n", world_rank,
            (double)m * n * 80 * 2 / 1e9);
    return 3;
  }
  Bert_Model<__half>* model = new Bert_Model<__half>(BertParams, SParams, k, n, workspace);

  const int ws = world_size, r = world_rank, H = k, Hl = H / ws, F = 4 * H, Fl = F / ws;
  const int M = batch * seq;
  for (int l = 0; l < layers; ++l) {
    Bert_Encoder<__half>* e = model->encoders[l];
    const uint32_t id0 = (uint32_t)l * 32u;
    fw(e->MHA->linear_q_col->weights, H, Hl, 0, r * Hl, H, id0 + W_Q, 0.0f, 0.02f);
    fw(e->MHA->linear_k_col->weights, H, Hl, 0, r * Hl, H, id0 + W_K, 0.0f, 0.02f);
    fw(e->MHA->linear_v_col->weights, H, Hl, 0, r * Hl, H, id0 + W_V, 0.0f, 0.02f);
    fw(e->MHA->linear_w_row->weights, Hl, H, r * Hl, 0, H, id0 + W_O, 0.0f, 0.02f);
    fw(e->MHA->q_bias, 1, Hl, 0, r * Hl, H, id0 + B_Q, 0.0f, 0.02f);
    fw(e->MHA->k_bias, 1, Hl, 0, r * Hl, H, id0 + B_K, 0.0f, 0.02f);
    fw(e->MHA->v_bias, 1, Hl, 0, r * Hl, H, id0 + B_V, 0.0f, 0.02f);
    fill_const<<<1184, 256>>>(e->MHA->attr_mask, (size_t)batch * seq * seq, 1.0f);
    fw(e->MLP->linear_col->weights, H, Fl, 0, r * Fl, F, id0 + W_UP, 0.0f, 0.02f);
    fw(e->MLP->linear_row->weights, Fl, H, r * Fl, 0, H, id0 + W_DOWN, 0.0f, 0.02f);
    fw(e->MLP->bias, 1, Fl, 0, r * Fl, F, id0 + B_UP, 0.0f, 0.02f);
    fw(e->ln_mha->gamma, 1, H, 0, 0, H, id0 + LN1_G, 1.0f, 0.02f);
    fw(e->ln_mha->beta, 1, H, 0, 0, H, id0 + LN1_B, 0.0f, 0.02f);
    fw(e->ln_mlp->gamma, 1, H, 0, 0, H, id0 + LN2_G, 1.0f, 0.02f);
    fw(e->ln_mlp->beta, 1, H, 0, 0, H, id0 + LN2_B, 0.0f, 0.02f);
  }
  fw(input, M, H, 0, 0, H, 0x10000u, 0.0f, 1.0f);
  if (cudaDeviceSynchronize() != cudaSuccess) { fprintf(stderr, "rank %d: fill failed\n", world_rank); return 3; }

  DynamicNvInitParam DParams;  // one stream + one cuBLAS handle
  std::vector<FuncWrap> vec = model->forward(input, output, batch, seq);
  auto step = [&]() { for (auto& f : vec) f.callback(DParams); };

  // host staging for the end-to-end variant (pinned)
  __half *hin = nullptr, *hout = nullptr;
  cudaHostAlloc((void**)&hin, sizeof(__half) * (size_t)M * H, cudaHostAllocDefault);
  cudaHostAlloc((void**)&hout, sizeof(__half) * (size_t)M * H, cudaHostAllocDefault);
  cudaMemcpy(hin, input, sizeof(__half) * (size_t)M * H, cudaMemcpyDeviceToHost);

  for (int i = 0; i < warmup; ++i) step();
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  cudaDeviceSynchronize();
  MPI_Barrier(MPI_COMM_WORLD);
  cudaEventRecord(e0, DParams.stream);
  for (int i = 0; i < steps; ++i) step();
  cudaEventRecord(e1, DParams.stream);
  cudaEventSynchronize(e1);
  float ms = 0.0f;
  cudaEventElapsedTime(&ms, e0, e1);
  MPI_Barrier(MPI_COMM_WORLD);

  // end to end: host input -> device, the pass, result -> host, every step (every rank needs the input)
  for (int i = 0; i < 2; ++i) {
    cudaMemcpyAsync(input, hin, sizeof(__half) * (size_t)M * H, cudaMemcpyHostToDevice, DParams.stream);
    step();
    cudaMemcpyAsync(hout, output, sizeof(__half) * (size_t)M * H, cudaMemcpyDeviceToHost, DParams.stream);
    cudaStreamSynchronize(DParams.stream);
  }
  MPI_Barrier(MPI_COMM_WORLD);
  cudaEventRecord(e0, DParams.stream);
  for (int i = 0; i < steps; ++i) {
    cudaMemcpyAsync(input, hin, sizeof(__half) * (size_t)M * H, cudaMemcpyHostToDevice, DParams.stream);
    step();
    cudaMemcpyAsync(hout, output, sizeof(__half) * (size_t)M * H, cudaMemcpyDeviceToHost, DParams.stream);
    cudaStreamSynchronize(DParams.stream);
  }
  cudaEventRecord(e1, DParams.stream);
  cudaEventSynchronize(e1);
  float ms_e2e = 0.0f;
  cudaEventElapsedTime(&ms_e2e, e0, e1);
  cudaError_t err = cudaDeviceSynchronize();
  MPI_Barrier(MPI_COMM_WORLD);

  if (dump && world_rank == 0) {
    FILE* f = fopen(dump, "wb");
    if (f) { fwrite(hout, sizeof(__half), (size_t)M * H, f); fclose(f); }
  }
  if (world_rank == 0) {
    printf("{\"ref_harness\": true, \"world_size\": %d, \"batch\": %d, \"seq\": %d, \"hidden\": %d, \"layers\": %d, "
           "\"kernels_per_step\": %zu, \"steps\": %d, \"ms_per_step\": %.6f, \"ms_per_step_e2e\": %.6f, "
           "\"tokens_per_s\": %.3f, \"tokens_per_s_e2e\": %.3f, \"cuda_error\": \"%s\"}\n",
           world_size, batch, seq, H, layers, vec.size(), steps, ms / steps, ms_e2e / steps,
           1000.0 * M * steps / ms, 1000.0 * M * steps / ms_e2e, cudaGetErrorString(err));
    fflush(stdout);
  }
  MPI_Finalize();
  return err == cudaSuccess ? 0 : 4;
}
