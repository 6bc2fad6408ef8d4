// Process <-> GPU binding and communicator bootstrap over MPI: the counterpart of the reference's
// createNcclComm (src/communicator.h:9-41).  Where the reference broadcasts one ncclUniqueId from
// rank 0, every rank here broadcasts the handle of its symmetric segment (world_size MPI_Bcast
// calls), after which all peer segments are mapped.
#pragma once
#include <cuda_runtime.h>
#include <mpi.h>

#include <cstdio>
#include <cstdlib>
#include <vector>

#include "context.h"
#include "scheduler.h"

namespace liger_host {

inline liger_comm* createLigerComm(int argc, char* argv[], int& world_size, int& world_rank, size_t data_bytes,
                                   int channels = 8) {
  int provided = 0;
  if (MPI_Init_thread(&argc, &argv, MPI_THREAD_MULTIPLE, &provided) != MPI_SUCCESS) {
    fprintf(stderr, "MPI_Init_thread failed\n");
    exit(2);
  }
  MPI_Comm_size(MPI_COMM_WORLD, &world_size);
  MPI_Comm_rank(MPI_COMM_WORLD, &world_rank);
  int device_count = 0;
  cudaGetDeviceCount(&device_count);
  if (device_count < world_size) {
    // the reference prints this and carries on (src/communicator.h:22-25); there is nothing useful to do then
    fprintf(stderr, "Error: This program requires at least %d GPUs (found %d)\n", world_size, device_count);
    MPI_Finalize();
    exit(2);
  }
  cudaSetDevice(world_rank);
  liger_comm* comm = nullptr;
  if (liger_comm_create(&comm, world_rank, world_size, data_bytes, channels) != LIGER_OK) {
    fprintf(stderr, "rank %d: liger_comm_create: %s\n", world_rank, liger_last_error());
    exit(2);
  }
  if (world_size > 1) {
    std::vector<unsigned char> all((size_t)world_size * LIGER_COMM_HANDLE_BYTES);
    liger_comm_export(comm, all.data() + (size_t)world_rank * LIGER_COMM_HANDLE_BYTES);
    for (int r = 0; r < world_size; ++r)
      MPI_Bcast(all.data() + (size_t)r * LIGER_COMM_HANDLE_BYTES, LIGER_COMM_HANDLE_BYTES, MPI_BYTE, r, MPI_COMM_WORLD);
    if (liger_comm_connect(comm, all.data()) != LIGER_OK) {
      fprintf(stderr, "rank %d: liger_comm_connect: %s\n", world_rank, liger_last_error());
      exit(2);
    }
    MPI_Barrier(MPI_COMM_WORLD);
  }
  printf("Communication Complete from Rank: %d\n", world_rank);
  return comm;
}

// Coordinator over the same MPI calls.
class MpiCoordinator : public Coordinator {
 public:
  MpiCoordinator(int rank, int size) : rank_(rank), size_(size) {}
  int rank() const override { return rank_; }
  int size() const override { return size_; }
  int broadcast_int(int v) override {
    MPI_Bcast(&v, 1, MPI_INT, 0, MPI_COMM_WORLD);
    return v;
  }
  void barrier() override { MPI_Barrier(MPI_COMM_WORLD); }

 private:
  int rank_, size_;
};

}  // namespace liger_host
