// Shared-memory implementation of the MPI subset declared in mpi.h (one node, one process per rank).
//
// Segment layout: a barrier (arrival counter + generation) and a broadcast mailbox (sequence
// number, acknowledgement counter, 64 KiB payload).  Barrier and broadcast keep separate state, so
// one thread may sit in MPI_Barrier while another broadcasts (the reference's request thread and
// scheduler thread do exactly that).  Waits yield the CPU and give up after a timeout
// (LIGER_MPI_TIMEOUT_S, default 300 s) with an error message instead of hanging a job.
#include "mpi.h"

#include <fcntl.h>
#include <sched.h>
#include <signal.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <time.h>
#include <unistd.h>

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cerrno>
#include <cstring>
#include <string>

namespace {

constexpr uint32_t kMagic = 0x4c4d5049u;
constexpr size_t kMailbox = 65536;

struct Segment {
  std::atomic<uint32_t> magic;
  std::atomic<int> creator_pid;  // rank 0 of the job that created the segment
  std::atomic<int> attached;
  std::atomic<int> bar_count;
  std::atomic<int> bar_gen;
  std::atomic<uint64_t> bc_seq;
  std::atomic<int> bc_acks;
  char pad[64];
  char mailbox[kMailbox];
};

Segment* g_seg = nullptr;
int g_rank = 0, g_size = 1;
uint64_t g_bc_seen = 0;
std::string g_name;
double g_timeout_s = 300.0;

int env_int(const char* const* names, int fallback) {
  for (int i = 0; names[i]; ++i) {
    const char* v = getenv(names[i]);
    if (v && *v) return atoi(v);
  }
  return fallback;
}

double now_s() {
  struct timespec ts;
  clock_gettime(CLOCK_MONOTONIC, &ts);
  return (double)ts.tv_sec + 1e-9 * (double)ts.tv_nsec;
}

template <typename Pred>
bool wait_until(Pred p, const char* what) {
  const double t0 = now_s();
  unsigned spins = 0;
  while (!p()) {
    if ((++spins & 0x3ff) == 0) {
      sched_yield();
      if (now_s() - t0 > g_timeout_s) {
        fprintf(stderr, "[liger mpi shim] rank %d: timeout after %.0f s in %s\n", g_rank, g_timeout_s, what);
        return false;
      }
    }
  }
  return true;
}

int dtype_size(MPI_Datatype t) {
  switch (t) {
    case MPI_BYTE: return 1;
    case MPI_INT: return 4;
    case MPI_FLOAT: return 4;
    case MPI_DOUBLE: return 8;
    default: return 1;
  }
}

}  // namespace

extern "C" {

int MPI_Init_thread(int*, char***, int required, int* provided) {
  if (provided) *provided = required;
  if (g_seg) return MPI_SUCCESS;
  static const char* const rank_names[] = {"LIGER_MPI_RANK", "OMPI_COMM_WORLD_RANK", "PMI_RANK", "RANK", nullptr};
  static const char* const size_names[] = {"LIGER_MPI_SIZE", "OMPI_COMM_WORLD_SIZE", "PMI_SIZE", "WORLD_SIZE", nullptr};
  g_rank = env_int(rank_names, 0);
  g_size = env_int(size_names, 1);
  if (const char* t = getenv("LIGER_MPI_TIMEOUT_S")) g_timeout_s = atof(t);
  if (g_size <= 1) { g_size = 1; g_rank = 0; return MPI_SUCCESS; }
  const char* job = getenv("LIGER_MPI_JOB");
  if (!job || !*job) job = getenv("MASTER_PORT");
  char buf[128];
  if (job && *job) snprintf(buf, sizeof(buf), "/liger_mpi_%s", job);
  else snprintf(buf, sizeof(buf), "/liger_mpi_ppid%d", (int)getppid());
  g_name = buf;
  // Rank 0 always replaces whatever segment of that name a previous (possibly crashed) job left
  // behind.  The other ranks may open the name before rank 0 got that far, so they verify what they
  // mapped: the creator must still be alive and the attach count must not exceed the world size;
  // otherwise they let go and look again.
  const double t_begin = now_s();
  for (;;) {
    int fd = -1;
    if (g_rank == 0) {
      shm_unlink(g_name.c_str());
      fd = shm_open(g_name.c_str(), O_CREAT | O_EXCL | O_RDWR, 0600);
      if (fd < 0 || ftruncate(fd, sizeof(Segment)) != 0) {
        perror("[liger mpi shim] shm_open/ftruncate");
        return MPI_ERR_OTHER;
      }
    } else {
      while ((fd = shm_open(g_name.c_str(), O_RDWR, 0600)) < 0) {
        usleep(1000);
        if (now_s() - t_begin > g_timeout_s) { fprintf(stderr, "[liger mpi shim] rank %d: no segment %s\n", g_rank, buf); return MPI_ERR_OTHER; }
      }
      struct stat st;
      while (fstat(fd, &st) == 0 && (size_t)st.st_size < sizeof(Segment)) {
        usleep(1000);
        if (now_s() - t_begin > g_timeout_s) return MPI_ERR_OTHER;
      }
    }
    void* p = mmap(nullptr, sizeof(Segment), PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
    close(fd);
    if (p == MAP_FAILED) { perror("[liger mpi shim] mmap"); return MPI_ERR_OTHER; }
    g_seg = (Segment*)p;
    if (g_rank == 0) {
      g_seg->creator_pid.store((int)getpid());
      g_seg->attached.store(1);
      g_seg->bar_count.store(0);
      g_seg->bar_gen.store(0);
      g_seg->bc_seq.store(0);
      g_seg->bc_acks.store(g_size - 1);
      g_seg->magic.store(kMagic, std::memory_order_release);
      break;
    }
    bool fresh = false;
    const double t_map = now_s();
    while (now_s() - t_map < 0.2) {  // give a just-created segment a moment to be initialised
      if (g_seg->magic.load(std::memory_order_acquire) == kMagic) { fresh = true; break; }
      usleep(200);
    }
    if (fresh) {
      const int pid = g_seg->creator_pid.load();
      const bool alive = pid > 0 && (kill(pid, 0) == 0 || errno == EPERM);
      if (alive && g_seg->attached.fetch_add(1) < g_size) break;  // ours
    }
    munmap(g_seg, sizeof(Segment));
    g_seg = nullptr;
    if (now_s() - t_begin > g_timeout_s) {
      fprintf(stderr, "[liger mpi shim] rank %d: only stale segments named %s\n", g_rank, buf);
      return MPI_ERR_OTHER;
    }
    usleep(2000);
  }
  if (!wait_until([] { return g_seg->attached.load() >= g_size; }, "MPI_Init (waiting for all ranks)")) return MPI_ERR_OTHER;
  return MPI_SUCCESS;
}

int MPI_Init(int* argc, char*** argv) { int p; return MPI_Init_thread(argc, argv, MPI_THREAD_SINGLE, &p); }

int MPI_Comm_size(MPI_Comm, int* size) { *size = g_size; return MPI_SUCCESS; }
int MPI_Comm_rank(MPI_Comm, int* rank) { *rank = g_rank; return MPI_SUCCESS; }

int MPI_Barrier(MPI_Comm) {
  if (g_size == 1 || !g_seg) return MPI_SUCCESS;
  const int gen = g_seg->bar_gen.load(std::memory_order_acquire);
  if (g_seg->bar_count.fetch_add(1, std::memory_order_acq_rel) == g_size - 1) {
    g_seg->bar_count.store(0, std::memory_order_relaxed);
    g_seg->bar_gen.store(gen + 1, std::memory_order_release);
    return MPI_SUCCESS;
  }
  return wait_until([gen] { return g_seg->bar_gen.load(std::memory_order_acquire) != gen; }, "MPI_Barrier") ? MPI_SUCCESS
                                                                                                             : MPI_ERR_OTHER;
}

int MPI_Bcast(void* buffer, int count, MPI_Datatype datatype, int root, MPI_Comm) {
  if (g_size == 1 || !g_seg) return MPI_SUCCESS;
  size_t left = (size_t)count * dtype_size(datatype);
  char* p = (char*)buffer;
  while (left > 0) {
    const size_t n = left < kMailbox ? left : kMailbox;
    if (g_rank == root) {
      if (!wait_until([] { return g_seg->bc_acks.load(std::memory_order_acquire) >= g_size - 1; }, "MPI_Bcast (root)"))
        return MPI_ERR_OTHER;
      g_seg->bc_acks.store(0, std::memory_order_relaxed);
      memcpy(g_seg->mailbox, p, n);
      g_bc_seen = g_seg->bc_seq.load(std::memory_order_relaxed) + 1;
      g_seg->bc_seq.store(g_bc_seen, std::memory_order_release);
    } else {
      const uint64_t want = g_bc_seen + 1;
      if (!wait_until([want] { return g_seg->bc_seq.load(std::memory_order_acquire) >= want; }, "MPI_Bcast (receiver)"))
        return MPI_ERR_OTHER;
      memcpy(p, g_seg->mailbox, n);
      g_bc_seen = want;
      g_seg->bc_acks.fetch_add(1, std::memory_order_acq_rel);
    }
    p += n;
    left -= n;
  }
  return MPI_SUCCESS;
}

int MPI_Finalize(void) {
  if (g_seg) {
    MPI_Barrier(MPI_COMM_WORLD);
    munmap(g_seg, sizeof(Segment));
    g_seg = nullptr;
    if (g_rank == 0) shm_unlink(g_name.c_str());
  }
  return MPI_SUCCESS;
}

}  // extern "C"
