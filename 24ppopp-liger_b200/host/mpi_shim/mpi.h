/*
 * A single-node stand-in for the six MPI calls the serving path uses (MPI_Init_thread,
 * MPI_Comm_size, MPI_Comm_rank, MPI_Bcast, MPI_Barrier, MPI_Finalize -- the reference's call sites
 * are src/communicator.h:13-35, src/schedule.h:288-296 and src/utils.h:298-299), for machines
 * without an MPI installation.  Ranks are processes of one node that share a POSIX shared-memory
 * segment; rank and size come from the environment (LIGER_MPI_RANK / LIGER_MPI_SIZE, or the
 * variables Open MPI, PMI and torchrun set).  With a real MPI installed, include its <mpi.h>
 * instead: the host code only uses these six calls.
 */
#ifndef LIGER_MPI_SHIM_H
#define LIGER_MPI_SHIM_H

#ifdef __cplusplus
extern "C" {
#endif

typedef int MPI_Comm;
typedef int MPI_Datatype;

#define MPI_COMM_WORLD 0
#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15

#define MPI_BYTE 1
#define MPI_CHAR 1
#define MPI_INT 4
#define MPI_FLOAT 5
#define MPI_DOUBLE 8

#define MPI_THREAD_SINGLE 0
#define MPI_THREAD_FUNNELED 1
#define MPI_THREAD_SERIALIZED 2
#define MPI_THREAD_MULTIPLE 3

int MPI_Init(int* argc, char*** argv);
int MPI_Init_thread(int* argc, char*** argv, int required, int* provided);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Bcast(void* buffer, int count, MPI_Datatype datatype, int root, MPI_Comm comm);
int MPI_Barrier(MPI_Comm comm);
int MPI_Finalize(void);

#ifdef __cplusplus
}
#endif
#endif
