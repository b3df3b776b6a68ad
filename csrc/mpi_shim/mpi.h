// Minimal single-host MPI for machines where no MPI is installed: enough for this library's MPI
// front door (homcomp_mpi.h) and for building the reference library (what
// HomComp/src/cuda_awareallreduce.cu uses).  Ranks are processes on one machine (started
// by torch.distributed.run or any launcher that sets RANK / WORLD_SIZE / MASTER_PORT); messages
// between device buffers travel GPU to GPU through persistent, IPC-mapped device mailboxes (what a
// CUDA-aware MPI does inside one node), matched in FIFO order per (source, destination) pair.
#pragma once
#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef int MPI_Info;
typedef struct MPI_Status_ {
  int MPI_SOURCE, MPI_TAG, MPI_ERROR;
  long long count_bytes;
} MPI_Status;
typedef struct hcref_request* MPI_Request;

#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_COMM_WORLD 0
#define MPI_COMM_NULL (-1)
#define MPI_BYTE 1
#define MPI_FLOAT 4
#define MPI_DOUBLE 8
#define MPI_INT 5
#define MPI_SUM 1
#define MPI_MIN 2
#define MPI_MAX 3
#define MPI_INFO_NULL 0
#define MPI_COMM_TYPE_SHARED 1
#define MPI_REQUEST_NULL ((MPI_Request)0)
#define MPI_STATUS_IGNORE ((MPI_Status*)0)
#define MPI_STATUSES_IGNORE ((MPI_Status*)0)
#define MPI_IN_PLACE ((void*)-1)
#define MPI_MAX_ERROR_STRING 256

int MPI_Init(int* argc, char*** argv);
int MPI_Finalize(void);
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Send(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm);
int MPI_Isend(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Irecv(void* buf, int count, MPI_Datatype dt, int source, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Wait(MPI_Request* req, MPI_Status* status);
int MPI_Waitall(int n, MPI_Request* reqs, MPI_Status* statuses);
int MPI_Sendrecv(const void* sbuf, int scount, MPI_Datatype sdt, int dest, int stag, void* rbuf, int rcount,
                 MPI_Datatype rdt, int source, int rtag, MPI_Comm comm, MPI_Status* status);
int MPI_Get_count(const MPI_Status* status, MPI_Datatype dt, int* count);
int MPI_Barrier(MPI_Comm comm);
double MPI_Wtime(void);
int MPI_Comm_split_type(MPI_Comm comm, int type, int key, MPI_Info info, MPI_Comm* newcomm);
int MPI_Comm_split(MPI_Comm comm, int color, int key, MPI_Comm* newcomm);
int MPI_Comm_free(MPI_Comm* comm);
int MPI_Error_string(int code, char* str, int* len);
int MPI_Abort(MPI_Comm comm, int code);

#ifdef __cplusplus
}
#endif
