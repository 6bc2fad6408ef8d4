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
//   liger_ref_harness ops <dump_dir>
//   liger_ref_harness sweep <max_megabytes> <steps>
//
// The third form times the reference's collective as it is bound in src/layer/linear.h:55-60 -- an in-place
// ncclAllReduce (src/layer/func_wrapper.h:40-43) -- followed by its residual kernel add_bias_input
// (src/cuda/cuda_kernels.cu:438-461) on fp16 tensors from 8 KB to <max_megabytes> MB in powers of two.
// The second form runs the reference's own kernels and its cuBLAS-backed linear layers one at a time
// on seeded inputs (tensor ids 0x20000 + ...) and writes each result as raw fp16 to
// <dump_dir>/<name>.f16, with a manifest of names and shapes on stdout: the per-operator vectors
// that pin the CPU oracle and this repository's kernels to the reference's own output.
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

// ---- per-operator vectors -----------------------------------------------------------------------------
static __half* dalloc(size_t n) {
  __half* p = nullptr;
  if (cudaMalloc((void**)&p, sizeof(__half) * (n ? n : 1)) != cudaSuccess) { fprintf(stderr, "cudaMalloc failed\n"); exit(3); }
  return p;
}
static __half* seeded(size_t rows, size_t cols, uint32_t id, float mean, float std) {
  __half* p = dalloc(rows * cols);
  fw(p, (int)rows, (int)cols, 0, 0, (int)cols, id, mean, std);
  return p;
}
static std::string g_dir;
static std::string g_manifest;
static void dump(const char* name, const __half* dev, std::initializer_list<int> shape) {
  size_t n = 1;
  for (int s : shape) n *= (size_t)s;
  std::vector<__half> h(n);
  if (cudaMemcpy(h.data(), dev, n * sizeof(__half), cudaMemcpyDeviceToHost) != cudaSuccess) {
    fprintf(stderr, "ops: copy of %s failed: %s\n", name, cudaGetErrorString(cudaGetLastError()));
    exit(4);
  }
  const std::string path = g_dir + "/" + name + ".f16";
  FILE* f = fopen(path.c_str(), "wb");
  if (!f || fwrite(h.data(), sizeof(__half), n, f) != n) { fprintf(stderr, "ops: cannot write %s\n", path.c_str()); exit(5); }
  fclose(f);
  if (!g_manifest.empty()) g_manifest += ", ";
  g_manifest += std::string("\"") + name + "\": [";
  bool first = true;
  for (int s : shape) { g_manifest += (first ? "" : ", ") + std::to_string(s); first = false; }
  g_manifest += "]";
}
// mask[b][q][k]: batch 0 causal (k <= q), other batches padding (the last quarter of the keys masked out)
__global__ void fill_mask(__half* mask, int B, int S) {
  const size_t total = (size_t)B * S * S;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const int k = (int)(i % S), q = (int)((i / S) % S), b = (int)(i / ((size_t)S * S));
    const bool keep = b == 0 ? k <= q : k < S - S / 4;
    mask[i] = __float2half(keep ? 1.0f : 0.0f);
  }
}

static int run_ops(const char* dir, const StaticNvInitParam& SParams) {
  g_dir = dir;
  DynamicNvInitParam DParams;
  cudaStream_t st = DParams.stream;
  {  // LayerNorm (src/cuda/cuda_kernels.cu:463-532), two widths
    const int shapes[2][2] = {{24, 1024}, {8, 12288}};
    for (int c = 0; c < 2; ++c) {
      const int m = shapes[c][0], n = shapes[c][1];
      const uint32_t id = 0x20000u + 8u * c;
      __half *x = seeded(m, n, id, 0.3f, 1.5f), *g = seeded(1, n, id + 1, 1.0f, 0.02f), *b = seeded(1, n, id + 2, 0.0f, 0.02f);
      __half* y = dalloc((size_t)m * n);
      layer_norm<__half>(x, g, b, y, m, n, st);
      cudaStreamSynchronize(st);
      dump(c == 0 ? "layernorm_1024" : "layernorm_12288", y, {m, n});
    }
  }
  {  // bias + GELU in place (src/cuda/cuda_kernels.cu:71-84,302-319)
    const int m = 40, n = 4096;
    __half *x = seeded(m, n, 0x20010u, 0.0f, 1.5f), *b = seeded(1, n, 0x20011u, 0.0f, 0.5f);
    add_bias_act_kernelLauncher<__half>(x, b, m, n, st);
    cudaStreamSynchronize(st);
    dump("bias_gelu", x, {m, n});
  }
  {  // bias + head split (src/cuda/attention_kernels.cu:133-163,226-329): k <= 1024 and k > 1024 launch paths
    const int cases[2][4] = {{2, 64, 4, 64}, {2, 64, 16, 128}};
    for (int c = 0; c < 2; ++c) {
      const int B = cases[c][0], S = cases[c][1], h = cases[c][2], D = cases[c][3], k = h * D, m = B * S;
      const uint32_t id = 0x20020u + 8u * c;
      __half *Q = seeded(m, k, id, 0.0f, 1.0f), *K = seeded(m, k, id + 1, 0.0f, 1.0f), *V = seeded(m, k, id + 2, 0.0f, 1.0f);
      __half *bq = seeded(1, k, id + 3, 0.0f, 0.5f), *bk = seeded(1, k, id + 4, 0.0f, 0.5f), *bv = seeded(1, k, id + 5, 0.0f, 0.5f);
      __half *qo = dalloc((size_t)m * k), *ko = dalloc((size_t)m * k), *vo = dalloc((size_t)m * k);
      add_QKV_bias_transpose_kernelLauncher<__half>(qo, ko, vo, Q, bq, K, bk, V, bv, B, S, h, D, st);
      cudaStreamSynchronize(st);
      const std::string tag = c == 0 ? "qkv_split_256" : "qkv_split_2048";
      dump((tag + "_q").c_str(), qo, {B, h, S, D});
      dump((tag + "_k").c_str(), ko, {B, h, S, D});
      dump((tag + "_v").c_str(), vo, {B, h, S, D});
    }
  }
  {  // scaled masked softmax in place (src/cuda/attention_kernels.cu:543-573,620-680)
    const int cases[2][3] = {{2, 4, 64}, {2, 2, 200}};
    for (int c = 0; c < 2; ++c) {
      const int B = cases[c][0], h = cases[c][1], S = cases[c][2];
      __half* s = seeded((size_t)B * h * S, S, 0x20030u + (uint32_t)c, 0.0f, 8.0f);
      __half* mask = dalloc((size_t)B * S * S);
      fill_mask<<<64, 256, 0, st>>>(mask, B, S);
      attn_softmax_kernelLauncher<__half>(s, mask, B, S, h, __float2half(0.125f), st);
      cudaStreamSynchronize(st);
      dump(c == 0 ? "softmax_64" : "softmax_200", s, {B, h, S, S});
    }
  }
  {  // head merge (src/cuda/attention_kernels.cu:693-742)
    const int B = 2, h = 4, S = 64, D = 64;
    __half* src = seeded((size_t)B * h * S, D, 0x20040u, 0.0f, 1.0f);
    __half* dst = dalloc((size_t)B * S * h * D);
    transpose_kernelLauncher<__half>(dst, src, B, S, h, D, st);
    cudaStreamSynchronize(st);
    dump("merge_heads", dst, {B * S, h * D});
  }
  {  // residual + bias + LayerNorm (src/cuda/cuda_kernels.cu:360-409) and residual + bias (:438-461)
    const int m = 24, n = 1024;
    __half *in = seeded(m, n, 0x20050u, 0.0f, 1.0f), *g = seeded(1, n, 0x20051u, 1.0f, 0.02f), *b = seeded(1, n, 0x20052u, 0.0f, 0.02f);
    __half *bias = seeded(1, n, 0x20053u, 0.0f, 0.5f), *out = seeded(m, n, 0x20054u, 0.0f, 1.0f), *norm = dalloc((size_t)m * n);
    add_bias_input_layernorm_2_kernelLauncher<__half>(in, g, b, bias, out, norm, m, n, st);
    cudaStreamSynchronize(st);
    dump("residual_ln_hidden", out, {m, n});
    dump("residual_ln_norm", norm, {m, n});
    __half *o2 = seeded(m, n, 0x20060u, 0.0f, 1.0f), *i2 = seeded(m, n, 0x20061u, 0.0f, 1.0f), *b2 = seeded(1, n, 0x20062u, 0.0f, 0.5f);
    add_bias_input_kernelLauncher<__half>(o2, b2, i2, m, n, st);
    cudaStreamSynchronize(st);
    dump("residual_add", o2, {m, n});
  }
  {  // the reference's linear layers = cublasGemmEx as bound in src/layer/linear.h:47-53,99-105
    const int m1 = 96, k1 = 1024, n1 = 512;
    Linear_Col<__half> col(SParams, k1, n1);
    fw(col.weights, k1, n1, 0, 0, n1, 0x20071u, 0.0f, 0.02f);
    __half *x1 = seeded(m1, k1, 0x20070u, 0.0f, 1.0f), *y1 = dalloc((size_t)m1 * n1);
    for (auto& f : col.forward(x1, y1, m1)) f.callback(DParams);
    cudaStreamSynchronize(st);
    dump("linear_col", y1, {m1, n1});
    const int m2 = 64, k2 = 4096, n2 = 1024;
    Linear_Row<__half> row(SParams, k2, n2);
    fw(row.weights, k2, n2, 0, 0, n2, 0x20073u, 0.0f, 0.02f);
    __half *x2 = seeded(m2, k2, 0x20072u, 0.0f, 1.0f), *y2 = dalloc((size_t)m2 * n2);
    for (auto& f : row.forward(x2, y2, m2)) f.callback(DParams);
    cudaStreamSynchronize(st);
    dump("linear_row", y2, {m2, n2});
  }
  const cudaError_t err = cudaDeviceSynchronize();
  printf("{\"ref_ops\": true, \"cuda_error\": \"%s\", \"tensors\": {%s}}\n", cudaGetErrorString(err), g_manifest.c_str());
  fflush(stdout);
  return err == cudaSuccess ? 0 : 4;
}

// ---- all-reduce + residual sweep ---------------------------------------------------------------------------
static int run_sweep(size_t max_bytes, int steps, const StaticNvInitParam& SParams) {
  DynamicNvInitParam DParams;
  cudaStream_t st = DParams.stream;
  const int ws = SParams.world_size, rank = SParams.world_rank;
  __half *output = dalloc(max_bytes / 2), *input = dalloc(max_bytes / 2), *bias = dalloc(8192);
  fill_const<<<64, 256, 0, st>>>(bias, 8192, 0.0f);
  cudaEvent_t e0, e1;
  cudaEventCreate(&e0); cudaEventCreate(&e1);
  std::string recs;
  for (size_t bytes = 8192; bytes <= max_bytes; bytes *= 2) {
    const int n = bytes >= ((size_t)1 << 20) ? 8192 : 1024;
    const int m = (int)(bytes / (2 * (size_t)n));
    fw(output, m, n, 0, 0, n, 600u + (uint32_t)rank, 0.0f, 1.0f);
    fw(input, m, n, 0, 0, n, 610u, 0.0f, 1.0f);
    int iters = steps * 4;
    if (bytes > ((size_t)64 << 20)) { iters = (int)(2000000000ull / bytes); if (iters > steps * 4) iters = steps * 4; if (iters < 3) iters = 3; }
    auto once = [&]() {
      Allreduce(output, output, (size_t)m * n, SParams.nccldatatype, ncclSum, SParams.comm, DParams);
      add_bias_input_kernelLauncher<__half>(output, bias, input, m, n, st);
    };
    for (int i = 0; i < 3; ++i) once();
    // (the reference reduces in place, so repeated launches overflow fp16 after a few sums; the time of neither
    // kernel depends on the values)
    cudaStreamSynchronize(st);
    cudaDeviceSynchronize();
    MPI_Barrier(MPI_COMM_WORLD);
    cudaEventRecord(e0, st);
    for (int i = 0; i < iters; ++i) once();
    cudaEventRecord(e1, st);
    cudaEventSynchronize(e1);
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    MPI_Barrier(MPI_COMM_WORLD);
    const double us = 1e3 * ms / iters;
    char buf[256];
    snprintf(buf, sizeof(buf), "%s{\"bytes\": %zu, \"rows\": %d, \"cols\": %d, \"us\": %.3f, \"bus_gbs\": %.3f, \"iters\": %d}",
             recs.empty() ? "" : ", ", bytes, m, n, us, 2.0 * (ws - 1) / ws * (double)bytes / (us * 1e-6) / 1e9, iters);
    recs += buf;
  }
  const cudaError_t err = cudaDeviceSynchronize();
  if (rank == 0) {
    printf("{\"ref_sweep\": true, \"world_size\": %d, \"cuda_error\": \"%s\", \"records\": [%s]}\n", ws, cudaGetErrorString(err),
           recs.c_str());
    fflush(stdout);
  }
  return err == cudaSuccess ? 0 : 4;
}

int main(int argc, char* argv[]) {
  if (argc == 3 && std::string(argv[1]) == "ops") {
    int ws = 1, wr = 0;
    ncclComm_t nc = createNcclComm(argc, argv, ws, wr);
    StaticNvInitParam SP(wr, ws, nc, 1);
    const int rc = ws == 1 ? run_ops(argv[2], SP) : 2;
    MPI_Finalize();
    return rc;
  }
  if (argc == 4 && std::string(argv[1]) == "sweep") {
    int ws = 1, wr = 0;
    ncclComm_t nc = createNcclComm(argc, argv, ws, wr);
    StaticNvInitParam SP(wr, ws, nc, 1);
    const int rc = run_sweep((size_t)atoi(argv[2]) << 20, atoi(argv[3]), SP);
    MPI_Finalize();
    return rc;
  }
  if (argc < 8) {
    fprintf(stderr, "usage: %s batch seq head_num size_per_head layers steps warmup [dump_file]\n       %s ops dump_dir\n       %s sweep max_megabytes steps\n", argv[0],
            argv[0], argv[0]);
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

  // end to end: host input -> device, the pass, result -> host, every step.  Every rank needs the whole
  // input (the reference has no way to distribute it); the result is replicated, so rank 0 alone downloads it.
  auto step_e2e = [&]() {
    cudaMemcpyAsync(input, hin, sizeof(__half) * (size_t)M * H, cudaMemcpyHostToDevice, DParams.stream);
    step();
    if (world_rank == 0)
      cudaMemcpyAsync(hout, output, sizeof(__half) * (size_t)M * H, cudaMemcpyDeviceToHost, DParams.stream);
    cudaStreamSynchronize(DParams.stream);
  };
  for (int i = 0; i < 2; ++i) step_e2e();
  MPI_Barrier(MPI_COMM_WORLD);
  cudaEventRecord(e0, DParams.stream);
  for (int i = 0; i < steps; ++i) step_e2e();
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
