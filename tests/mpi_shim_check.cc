// Exercises the six MPI calls of the shim the way the serving path uses them: a handle exchange by
// one broadcast per rank, barriers from a second thread while the main thread broadcasts, and a
// long run of small broadcasts (the scheduler's per-segment admission counts).
#include <mpi.h>

#include <cstdio>
#include <cstring>
#include <thread>
#include <vector>

int main(int argc, char** argv) {
  int provided = 0;
  if (MPI_Init_thread(&argc, &argv, MPI_THREAD_MULTIPLE, &provided) != MPI_SUCCESS) return 3;
  int size = 0, rank = -1;
  MPI_Comm_size(MPI_COMM_WORLD, &size);
  MPI_Comm_rank(MPI_COMM_WORLD, &rank);
  // 1. handle exchange: every rank broadcasts a 128-byte blob (host/communicator.h)
  std::vector<unsigned char> all((size_t)size * 128);
  for (int i = 0; i < 128; ++i) all[(size_t)rank * 128 + i] = (unsigned char)(rank * 7 + i);
  for (int r = 0; r < size; ++r) MPI_Bcast(all.data() + (size_t)r * 128, 128, MPI_BYTE, r, MPI_COMM_WORLD);
  for (int r = 0; r < size; ++r)
    for (int i = 0; i < 128; ++i)
      if (all[(size_t)r * 128 + i] != (unsigned char)(r * 7 + i)) { printf("rank %d: blob %d corrupt\n", rank, r); return 4; }
  MPI_Barrier(MPI_COMM_WORLD);
  // 2. a payload larger than the mailbox
  std::vector<int> big(100000);
  if (rank == 0) for (size_t i = 0; i < big.size(); ++i) big[i] = (int)(i * 31 + 5);
  MPI_Bcast(big.data(), (int)big.size(), MPI_INT, 0, MPI_COMM_WORLD);
  for (size_t i = 0; i < big.size(); ++i) if (big[i] != (int)(i * 31 + 5)) { printf("rank %d: big payload corrupt\n", rank); return 5; }
  // 3. barriers on a second thread while this thread broadcasts (src/schedule.h:291,296 vs the admission counts)
  std::thread t([&] { for (int i = 0; i < 200; ++i) MPI_Barrier(MPI_COMM_WORLD); });
  long sum = 0;
  for (int i = 0; i < 5000; ++i) {
    int v = rank == 0 ? i * 3 + 1 : -1;
    MPI_Bcast(&v, 1, MPI_INT, 0, MPI_COMM_WORLD);
    if (v != i * 3 + 1) { printf("rank %d: bcast %d got %d\n", rank, i, v); return 6; }
    sum += v;
  }
  t.join();
  MPI_Finalize();
  printf("rank %d of %d ok %ld\n", rank, size, sum);
  return 0;
}
