// liger_mpirun -np N program [args...]: starts N copies of `program` on this node with the
// environment the MPI shim reads (LIGER_MPI_RANK, LIGER_MPI_SIZE, LIGER_MPI_JOB), waits for all of
// them and returns the largest exit status.  Stands in for `mpirun -np N` (README of the reference)
// on machines without an MPI installation.
#include <sys/types.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

int main(int argc, char** argv) {
  int np = 1, first = 1;
  if (argc >= 3 && (!strcmp(argv[1], "-np") || !strcmp(argv[1], "-n"))) { np = atoi(argv[2]); first = 3; }
  if (np < 1 || first >= argc) {
    fprintf(stderr, "usage: liger_mpirun -np N program [args...]\n");
    return 2;
  }
  const std::string job = std::to_string((long)getpid());
  std::vector<pid_t> kids;
  for (int r = 0; r < np; ++r) {
    pid_t pid = fork();
    if (pid < 0) { perror("fork"); return 2; }
    if (pid == 0) {
      setenv("LIGER_MPI_RANK", std::to_string(r).c_str(), 1);
      setenv("LIGER_MPI_SIZE", std::to_string(np).c_str(), 1);
      setenv("LIGER_MPI_JOB", job.c_str(), 1);
      execvp(argv[first], argv + first);
      perror("execvp");
      _exit(127);
    }
    kids.push_back(pid);
  }
  int worst = 0;
  for (pid_t pid : kids) {
    int st = 0;
    waitpid(pid, &st, 0);
    int code = WIFEXITED(st) ? WEXITSTATUS(st) : 128 + (WIFSIGNALED(st) ? WTERMSIG(st) : 0);
    if (code > worst) worst = code;
  }
  return worst;
}
