/* MPI-shaped C interface over the library: the five calls the reference offers
 * (include/stdml/mpi.h:24-31), with the datatype and the operator honoured
 * (the reference's MPI_Allreduce always sums floats, src/stdml/collective/mpi.cpp:40-42)
 * and a few more datatypes / operators / calls.  Buffers may be host or CUDA
 * device memory.  Ranks come from the environment: OMPI_COMM_WORLD_*, KungFu or
 * torchrun variables. */
#ifndef STDML_MPI_H
#define STDML_MPI_H
#ifdef __cplusplus
extern "C" {
#endif

enum mpi_comm_t {
    MPI_COMM_WORLD,
};
typedef enum mpi_comm_t MPI_Comm;

enum mpi_datatype_t {
    MPI_FLOAT,
    MPI_DOUBLE,
    MPI_INT,
    MPI_LONG_LONG,
    MPI_UNSIGNED,
    MPI_UNSIGNED_LONG_LONG,
    MPI_CHAR,
    MPI_BYTE,
    MPI_SHORT,
};
typedef enum mpi_datatype_t MPI_Datatype;

enum mpi_op_t {
    MPI_SUM,
    MPI_MIN,
    MPI_MAX,
    MPI_PROD,
    MPI_BXOR,
};
typedef enum mpi_op_t MPI_Op;

#define MPI_SUCCESS 0
#define MPI_ERR_OTHER 15
/* sendbuf of MPI_Allreduce / MPI_Reduce: the operand is already in recvbuf */
#define MPI_IN_PLACE ((void *)1)
#define MPI_MAX_PROCESSOR_NAME 64

typedef struct mpi_status_t {
    int MPI_SOURCE;
    int MPI_TAG;
    int MPI_ERROR;
} MPI_Status;
#define MPI_STATUS_IGNORE ((MPI_Status *)0)

extern int MPI_Init(int *argc, char ***argv);
extern int MPI_Finalize(void);

extern int MPI_Comm_rank(MPI_Comm comm, int *p);
extern int MPI_Comm_size(MPI_Comm comm, int *p);

extern int MPI_Allreduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype datatype,
                         MPI_Op op, MPI_Comm comm);
/* beyond the reference */
extern int MPI_Barrier(MPI_Comm comm);
extern int MPI_Bcast(void *buffer, int count, MPI_Datatype datatype, int root, MPI_Comm comm);
extern int MPI_Allgather(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf,
                         int recvcount, MPI_Datatype recvtype, MPI_Comm comm);
extern int MPI_Reduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype datatype,
                      MPI_Op op, int root, MPI_Comm comm);
/* recvbuf matters on root only */
extern int MPI_Gather(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf,
                      int recvcount, MPI_Datatype recvtype, int root, MPI_Comm comm);
/* a message is matched by (source, tag); a send does not wait for its receive */
extern int MPI_Send(const void *buf, int count, MPI_Datatype datatype, int dest, int tag,
                    MPI_Comm comm);
extern int MPI_Recv(void *buf, int count, MPI_Datatype datatype, int source, int tag,
                    MPI_Comm comm, MPI_Status *status);
extern int MPI_Initialized(int *flag);
extern int MPI_Finalized(int *flag);
extern int MPI_Abort(MPI_Comm comm, int errorcode);
extern int MPI_Get_processor_name(char *name, int *resultlen);
extern double MPI_Wtime(void);
#ifdef __cplusplus
}
#endif
#endif
