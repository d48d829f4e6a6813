/*
 * mpi.h of a small single-node MPI stand-in ("mpi_shim").
 *
 * Purpose: let the unmodified llnl/Aluminum sources configure, compile and run on a
 * machine that has no MPI installation, so that its NCCL backend can be timed as the
 * baseline.  Aluminum uses MPI as its control plane (MPI_Init_thread, communicator
 * duplication / splitting, the broadcast of the NCCL unique id: src/mpi_impl.cpp:148-205,
 * include/aluminum/mpi_comm_and_stream_wrapper.hpp:50-65, src/nccl_impl.cpp:52-59 of the
 * reference) and its headers name about a hundred MPI symbols; all of them are declared
 * here and implemented in mpi_shim.cpp over Unix-domain sockets between the processes of
 * one machine.  Ranks come from the launcher's environment (RANK / WORLD_SIZE as set by
 * torchrun, or MPISHIM_RANK / MPISHIM_SIZE); a process without them is a world of one.
 *
 * This is not a general MPI: datatypes are the contiguous basic ones, there are no
 * wildcards (MPI_ANY_SOURCE / MPI_ANY_TAG), no derived datatypes, no one-sided
 * operations, no files, one node only.  It does not use and is not linked into the
 * aluminum-b200 library.
 */
#ifndef AL_BASELINE_MPI_SHIM_MPI_H
#define AL_BASELINE_MPI_SHIM_MPI_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MPI_VERSION 3
#define MPI_SUBVERSION 1
#define MPISHIM 1

typedef int MPI_Comm;
typedef int MPI_Datatype;
typedef int MPI_Op;
typedef int MPI_Request;
typedef int MPI_Group;
typedef int MPI_Info;
typedef int MPI_Errhandler;
typedef ptrdiff_t MPI_Aint;
typedef long long MPI_Count;
typedef long long MPI_Offset;

typedef struct MPI_Status {
  int MPI_SOURCE;
  int MPI_TAG;
  int MPI_ERROR;
  long long shim_bytes;
} MPI_Status;

#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
#define MPI_ERR_ARG 12
#define MPI_ERR_COMM 5

#define MPI_COMM_NULL ((MPI_Comm)0)
#define MPI_COMM_WORLD ((MPI_Comm)1)
#define MPI_COMM_SELF ((MPI_Comm)2)
#define MPI_GROUP_NULL ((MPI_Group)0)
#define MPI_GROUP_EMPTY ((MPI_Group)1)
#define MPI_REQUEST_NULL ((MPI_Request)0)
#define MPI_INFO_NULL ((MPI_Info)0)
#define MPI_OP_NULL ((MPI_Op)0)
#define MPI_DATATYPE_NULL ((MPI_Datatype)0)
#define MPI_ERRORS_ARE_FATAL ((MPI_Errhandler)1)
#define MPI_ERRORS_RETURN ((MPI_Errhandler)2)

#define MPI_STATUS_IGNORE ((MPI_Status*)0)
#define MPI_STATUSES_IGNORE ((MPI_Status*)0)
#define MPI_IN_PLACE ((void*)-1)
#define MPI_BOTTOM ((void*)0)
#define MPI_PROC_NULL (-2)
#define MPI_ANY_SOURCE (-3)
#define MPI_ANY_TAG (-4)
#define MPI_ROOT (-5)
#define MPI_UNDEFINED (-32766)
#define MPI_MAX_PROCESSOR_NAME 256
#define MPI_MAX_ERROR_STRING 256
#define MPI_MAX_LIBRARY_VERSION_STRING 256

#define MPI_THREAD_SINGLE 0
#define MPI_THREAD_FUNNELED 1
#define MPI_THREAD_SERIALIZED 2
#define MPI_THREAD_MULTIPLE 3

#define MPI_COMM_TYPE_SHARED 1
#define MPI_TAG_UB 1
#define MPI_IDENT 0
#define MPI_CONGRUENT 1
#define MPI_SIMILAR 2
#define MPI_UNEQUAL 3

/* datatypes: handle = small integer, see mpi_shim.cpp for sizes and kinds */
#define MPI_CHAR ((MPI_Datatype)1)
#define MPI_SIGNED_CHAR ((MPI_Datatype)2)
#define MPI_UNSIGNED_CHAR ((MPI_Datatype)3)
#define MPI_BYTE ((MPI_Datatype)4)
#define MPI_SHORT ((MPI_Datatype)5)
#define MPI_UNSIGNED_SHORT ((MPI_Datatype)6)
#define MPI_INT ((MPI_Datatype)7)
#define MPI_UNSIGNED ((MPI_Datatype)8)
#define MPI_LONG ((MPI_Datatype)9)
#define MPI_UNSIGNED_LONG ((MPI_Datatype)10)
#define MPI_LONG_LONG_INT ((MPI_Datatype)11)
#define MPI_LONG_LONG MPI_LONG_LONG_INT
#define MPI_UNSIGNED_LONG_LONG ((MPI_Datatype)12)
#define MPI_FLOAT ((MPI_Datatype)13)
#define MPI_DOUBLE ((MPI_Datatype)14)
#define MPI_LONG_DOUBLE ((MPI_Datatype)15)
#define MPI_INT8_T ((MPI_Datatype)16)
#define MPI_UINT8_T ((MPI_Datatype)17)
#define MPI_INT16_T ((MPI_Datatype)18)
#define MPI_UINT16_T ((MPI_Datatype)19)
#define MPI_INT32_T ((MPI_Datatype)20)
#define MPI_UINT32_T ((MPI_Datatype)21)
#define MPI_INT64_T ((MPI_Datatype)22)
#define MPI_UINT64_T ((MPI_Datatype)23)
#define MPI_C_BOOL ((MPI_Datatype)24)
#define MPI_CXX_BOOL ((MPI_Datatype)25)
#define MPI_WCHAR ((MPI_Datatype)26)
#define MPI_AINT ((MPI_Datatype)27)
#define MPI_COUNT ((MPI_Datatype)28)
#define MPI_OFFSET ((MPI_Datatype)29)

/* reduction operators */
#define MPI_SUM ((MPI_Op)1)
#define MPI_PROD ((MPI_Op)2)
#define MPI_MIN ((MPI_Op)3)
#define MPI_MAX ((MPI_Op)4)
#define MPI_LAND ((MPI_Op)5)
#define MPI_LOR ((MPI_Op)6)
#define MPI_LXOR ((MPI_Op)7)
#define MPI_BAND ((MPI_Op)8)
#define MPI_BOR ((MPI_Op)9)
#define MPI_BXOR ((MPI_Op)10)

typedef void MPI_User_function(void* invec, void* inoutvec, int* len, MPI_Datatype* datatype);

/* environment */
int MPI_Init(int* argc, char*** argv);
int MPI_Init_thread(int* argc, char*** argv, int required, int* provided);
int MPI_Query_thread(int* provided);
int MPI_Initialized(int* flag);
int MPI_Finalized(int* flag);
int MPI_Finalize(void);
int MPI_Abort(MPI_Comm comm, int errorcode);
double MPI_Wtime(void);
int MPI_Get_processor_name(char* name, int* resultlen);
int MPI_Get_version(int* version, int* subversion);
int MPI_Get_library_version(char* version, int* resultlen);
int MPI_Error_string(int errorcode, char* string, int* resultlen);
int MPI_Comm_set_errhandler(MPI_Comm comm, MPI_Errhandler errhandler);

/* communicators and groups */
int MPI_Comm_rank(MPI_Comm comm, int* rank);
int MPI_Comm_size(MPI_Comm comm, int* size);
int MPI_Comm_dup(MPI_Comm comm, MPI_Comm* newcomm);
int MPI_Comm_split(MPI_Comm comm, int color, int key, MPI_Comm* newcomm);
int MPI_Comm_split_type(MPI_Comm comm, int split_type, int key, MPI_Info info, MPI_Comm* newcomm);
int MPI_Comm_create(MPI_Comm comm, MPI_Group group, MPI_Comm* newcomm);
int MPI_Comm_free(MPI_Comm* comm);
int MPI_Comm_get_attr(MPI_Comm comm, int keyval, void* attribute_val, int* flag);
int MPI_Comm_compare(MPI_Comm a, MPI_Comm b, int* result);
int MPI_Comm_group(MPI_Comm comm, MPI_Group* group);
int MPI_Group_size(MPI_Group group, int* size);
int MPI_Group_rank(MPI_Group group, int* rank);
int MPI_Group_incl(MPI_Group group, int n, const int ranks[], MPI_Group* newgroup);
int MPI_Group_translate_ranks(MPI_Group g1, int n, const int ranks1[], MPI_Group g2, int ranks2[]);
int MPI_Group_free(MPI_Group* group);

/* datatypes and operators */
int MPI_Type_size(MPI_Datatype datatype, int* size);
int MPI_Get_count(const MPI_Status* status, MPI_Datatype datatype, int* count);
int MPI_Op_create(MPI_User_function* fn, int commute, MPI_Op* op);
int MPI_Op_free(MPI_Op* op);

/* point to point */
int MPI_Send(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm);
int MPI_Recv(void* buf, int count, MPI_Datatype dt, int source, int tag, MPI_Comm comm, MPI_Status* status);
int MPI_Isend(const void* buf, int count, MPI_Datatype dt, int dest, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Irecv(void* buf, int count, MPI_Datatype dt, int source, int tag, MPI_Comm comm, MPI_Request* req);
int MPI_Sendrecv(const void* sendbuf, int sendcount, MPI_Datatype sendtype, int dest, int sendtag, void* recvbuf,
                 int recvcount, MPI_Datatype recvtype, int source, int recvtag, MPI_Comm comm, MPI_Status* status);
int MPI_Sendrecv_replace(void* buf, int count, MPI_Datatype dt, int dest, int sendtag, int source, int recvtag,
                         MPI_Comm comm, MPI_Status* status);
int MPI_Isendrecv(const void* sendbuf, int sendcount, MPI_Datatype sendtype, int dest, int sendtag, void* recvbuf,
                  int recvcount, MPI_Datatype recvtype, int source, int recvtag, MPI_Comm comm, MPI_Request* req);
int MPI_Wait(MPI_Request* req, MPI_Status* status);
int MPI_Test(MPI_Request* req, int* flag, MPI_Status* status);
int MPI_Waitall(int count, MPI_Request reqs[], MPI_Status statuses[]);
int MPI_Testall(int count, MPI_Request reqs[], int* flag, MPI_Status statuses[]);
int MPI_Request_free(MPI_Request* req);

/* collectives, blocking */
int MPI_Barrier(MPI_Comm comm);
int MPI_Bcast(void* buf, int count, MPI_Datatype dt, int root, MPI_Comm comm);
int MPI_Reduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm);
int MPI_Allreduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm);
int MPI_Reduce_scatter(const void* sendbuf, void* recvbuf, const int recvcounts[], MPI_Datatype dt, MPI_Op op,
                       MPI_Comm comm);
int MPI_Reduce_scatter_block(const void* sendbuf, void* recvbuf, int recvcount, MPI_Datatype dt, MPI_Op op,
                             MPI_Comm comm);
int MPI_Allgather(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
                  MPI_Datatype recvtype, MPI_Comm comm);
int MPI_Allgatherv(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, const int recvcounts[],
                   const int displs[], MPI_Datatype recvtype, MPI_Comm comm);
int MPI_Gather(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
               MPI_Datatype recvtype, int root, MPI_Comm comm);
int MPI_Gatherv(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, const int recvcounts[],
                const int displs[], MPI_Datatype recvtype, int root, MPI_Comm comm);
int MPI_Scatter(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
                MPI_Datatype recvtype, int root, MPI_Comm comm);
int MPI_Scatterv(const void* sendbuf, const int sendcounts[], const int displs[], MPI_Datatype sendtype,
                 void* recvbuf, int recvcount, MPI_Datatype recvtype, int root, MPI_Comm comm);
int MPI_Alltoall(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
                 MPI_Datatype recvtype, MPI_Comm comm);
int MPI_Alltoallv(const void* sendbuf, const int sendcounts[], const int sdispls[], MPI_Datatype sendtype,
                  void* recvbuf, const int recvcounts[], const int rdispls[], MPI_Datatype recvtype, MPI_Comm comm);

/* collectives, non-blocking */
int MPI_Ibarrier(MPI_Comm comm, MPI_Request* req);
int MPI_Ibcast(void* buf, int count, MPI_Datatype dt, int root, MPI_Comm comm, MPI_Request* req);
int MPI_Ireduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype dt, MPI_Op op, int root, MPI_Comm comm,
                MPI_Request* req);
int MPI_Iallreduce(const void* sendbuf, void* recvbuf, int count, MPI_Datatype dt, MPI_Op op, MPI_Comm comm,
                   MPI_Request* req);
int MPI_Ireduce_scatter(const void* sendbuf, void* recvbuf, const int recvcounts[], MPI_Datatype dt, MPI_Op op,
                        MPI_Comm comm, MPI_Request* req);
int MPI_Ireduce_scatter_block(const void* sendbuf, void* recvbuf, int recvcount, MPI_Datatype dt, MPI_Op op,
                              MPI_Comm comm, MPI_Request* req);
int MPI_Iallgather(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
                   MPI_Datatype recvtype, MPI_Comm comm, MPI_Request* req);
int MPI_Iallgatherv(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf,
                    const int recvcounts[], const int displs[], MPI_Datatype recvtype, MPI_Comm comm,
                    MPI_Request* req);
int MPI_Igather(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
                MPI_Datatype recvtype, int root, MPI_Comm comm, MPI_Request* req);
int MPI_Igatherv(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, const int recvcounts[],
                 const int displs[], MPI_Datatype recvtype, int root, MPI_Comm comm, MPI_Request* req);
int MPI_Iscatter(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
                 MPI_Datatype recvtype, int root, MPI_Comm comm, MPI_Request* req);
int MPI_Iscatterv(const void* sendbuf, const int sendcounts[], const int displs[], MPI_Datatype sendtype,
                  void* recvbuf, int recvcount, MPI_Datatype recvtype, int root, MPI_Comm comm, MPI_Request* req);
int MPI_Ialltoall(const void* sendbuf, int sendcount, MPI_Datatype sendtype, void* recvbuf, int recvcount,
                  MPI_Datatype recvtype, MPI_Comm comm, MPI_Request* req);
int MPI_Ialltoallv(const void* sendbuf, const int sendcounts[], const int sdispls[], MPI_Datatype sendtype,
                   void* recvbuf, const int recvcounts[], const int rdispls[], MPI_Datatype recvtype, MPI_Comm comm,
                   MPI_Request* req);

#ifdef __cplusplus
}
#endif

#endif /* AL_BASELINE_MPI_SHIM_MPI_H */
