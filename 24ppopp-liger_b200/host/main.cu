// liger_main: the serving executable -- the counterpart of the reference's main.cu.
//
//   liger_mpirun -np N ./liger_main max_batch max_seq head_num size_per_head layer_num kernel_num factor arr_rate
//                [--mode profile,schedule,no_schedule] [--graph ref|preln] [--act gelu|geglu] [--ffn F]
//                [--causal 0|1] [--requests R] [--ignore I] [--poisson 0|1] [--seed S] [--seq-round Q]
//                [--min-seq L] [--contention C|auto] [--min-slice-eff E] [--depth D]
//
// The eight positional integers are the reference's (its argv parsing is commented out and the
// values hard-coded, main.cu:14-31; defaults here are the same: 2 128 128 96 4 16 8 80).  kernel_num is
// accepted for command-line compatibility; this implementation's fused layer has 7 kernels
// whatever is passed.  Without --mode the three entry points run in the reference's order
// (profile, schedule, no_schedule; main.cu:49-53).
#define LIGER_HOST_WITH_CUDA 1
#include <mpi.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include "communicator.h"
#include "layers.h"
#include "test_schedule.h"

using namespace liger_host;

int main(int argc, char* argv[]) {
  int vals[8] = {2, 128, 128, 96, 4, 16, 8, 80};
  int npos = 0;
  std::string mode = "profile,schedule,no_schedule";
  BertInitParam bp;
  for (int i = 1; i < argc; ++i) {
    const std::string a = argv[i];
    auto next = [&](const char* what) -> const char* {
      if (i + 1 >= argc) { fprintf(stderr, "missing value for %s\n", what); exit(2); }
      return argv[++i];
    };
    if (a == "--mode") mode = next("--mode");
    else if (a == "--graph") { const std::string v = next("--graph"); bp.graph = (v == "preln" || v == "1") ? GRAPH_PRELN : GRAPH_REF; }
    else if (a == "--act") { const std::string v = next("--act"); bp.act = (v == "geglu" || v == "1") ? ACT_GEGLU : ACT_GELU; }
    else if (a == "--ffn") bp.ffn_inner = atoi(next("--ffn"));
    else if (a == "--causal") bp.causal = atoi(next("--causal"));
    else if (a == "--requests") bp.num_requests = atoi(next("--requests"));
    else if (a == "--ignore") bp.ignore_num = atoi(next("--ignore"));
    else if (a == "--poisson") bp.poisson = atoi(next("--poisson"));
    else if (a == "--seed") bp.seed = (uint32_t)atoi(next("--seed"));
    else if (a == "--seq-round") bp.seq_round = atoi(next("--seq-round"));
    else if (a == "--min-seq") bp.min_seq_len = atoi(next("--min-seq"));
    else if (a == "--contention") { const std::string v = next("--contention"); bp.contention = v == "auto" ? 0.0f : (float)atof(v.c_str()); }
    else if (a == "--min-slice-eff") bp.min_slice_efficiency = (float)atof(next("--min-slice-eff"));
    else if (a == "--depth") { bp.schedule_deep = atoi(next("--depth")); bp.workspace_slots = bp.schedule_deep + 1; }
    else if (a[0] != '-' && npos < 8) vals[npos++] = atoi(a.c_str());
    else { fprintf(stderr, "unknown argument %s\n", a.c_str()); return 2; }
  }
  if (npos != 0 && npos != 8) { fprintf(stderr, "give all eight positional integers or none\n"); return 2; }
  bp.max_batch_size = vals[0]; bp.max_seq_len = vals[1]; bp.head_num = vals[2]; bp.size_per_head = vals[3];
  bp.layer_num = vals[4]; bp.kernel_num = kKernelsPerLayer; bp.factor = vals[6];
  const int arr_rate = vals[7] > 0 ? vals[7] : 1;
  bp.rq_interval = (int)(1e6 / arr_rate);  // microseconds (main.cu:33)

  int world_size = 1, world_rank = 0;
  // the communicator must be sized before MPI tells us the world size: probe it from the environment
  // the same way the shim does, falling back to a size that fits any world
  const size_t comm_bytes = Bert_Model::comm_bytes_needed(bp);
  liger_comm* comm = createLigerComm(argc, argv, world_size, world_rank, comm_bytes, bp.workspace_slots);
  if (world_rank == 0 && vals[5] != kKernelsPerLayer)
    printf("note: kernel_num %d ignored; this implementation's layer has %d kernels\n", vals[5], kKernelsPerLayer);

  StaticNvInitParam staticNvParam(world_rank, world_size, comm, 1);
  CudaRuntime rt;
  MpiCoordinator coord(world_rank, world_size);
  EntryContext ctx{&rt, &coord};
  int rc = 0;
  try {
    size_t pos = 0;
    while (pos <= mode.size()) {
      size_t comma = mode.find(',', pos);
      if (comma == std::string::npos) comma = mode.size();
      const std::string m = mode.substr(pos, comma - pos);
      pos = comma + 1;
      if (m.empty()) continue;
      coord.barrier();
      if (m == "profile") test_profile(ctx, bp, staticNvParam);          // to collect profiling results
      else if (m == "schedule") test_schedule(ctx, bp, staticNvParam);   // running with Liger
      else if (m == "no_schedule") test_no_schedule(ctx, bp, staticNvParam);  // running without Liger
      else { fprintf(stderr, "unknown mode %s\n", m.c_str()); rc = 2; break; }
    }
  } catch (const std::exception& e) {
    fprintf(stderr, "rank %d: %s\n", world_rank, e.what());
    rc = 1;
  }
  unsigned int st[4];
  if (liger_device_status(st) != 0) {
    fprintf(stderr, "rank %d: device status %u at %#x (%u, %u)\n", world_rank, st[0], st[1], st[2], st[3]);
    rc = 1;
  }
  MPI_Finalize();
  return rc;
}
