#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>

#include <unistd.h>
#include <exception>
#include <memory>

#include <stdml/bits/collective/peer.hpp>
#include <stdml/mpi.h>

namespace sc = stdml::collective;

namespace
{
std::unique_ptr<sc::peer> g_peer;
std::unique_ptr<sc::session> g_sess;
bool g_finalized = false;

bool to_dtype(MPI_Datatype t, sc::dtype &out)
{
    switch (t) {
    case MPI_FLOAT:
        out = sc::f32;
        return true;
    case MPI_DOUBLE:
        out = sc::f64;
        return true;
    case MPI_INT:
        out = sc::i32;
        return true;
    case MPI_LONG_LONG:
        out = sc::i64;
        return true;
    case MPI_UNSIGNED:
        out = sc::u32;
        return true;
    case MPI_UNSIGNED_LONG_LONG:
        out = sc::u64;
        return true;
    case MPI_CHAR:
        out = sc::i8;
        return true;
    case MPI_BYTE:
        out = sc::u8;
        return true;
    case MPI_SHORT:
        out = sc::i16;
        return true;
    }
    return false;
}

bool to_op(MPI_Op o, sc::reduce_op &out)
{
    switch (o) {
    case MPI_SUM:
        out = sc::sum;
        return true;
    case MPI_MIN:
        out = sc::min;
        return true;
    case MPI_MAX:
        out = sc::max;
        return true;
    case MPI_PROD:
        out = sc::prod;
        return true;
    case MPI_BXOR:
        out = sc::bit_xor;
        return true;
    }
    return false;
}

template <typename F>
int guarded(F f)
{
    if (!g_sess) { return MPI_ERR_OTHER; }
    try {
        f();
        return MPI_SUCCESS;
    } catch (const std::exception &e) {
        std::fprintf(stderr, "stdml mpi: %s\n", e.what());
        return MPI_ERR_OTHER;
    }
}
}  // namespace

extern "C" {
int MPI_Init(int *, char ***)
{
    if (g_sess) { return MPI_SUCCESS; }
    try {
        g_peer = std::make_unique<sc::peer>(sc::peer::from_env());
        g_sess = g_peer->join_elastic();
        return MPI_SUCCESS;
    } catch (const std::exception &e) {
        std::fprintf(stderr, "stdml mpi: MPI_Init: %s\n", e.what());
        return MPI_ERR_OTHER;
    }
}

int MPI_Finalize(void)
{
    g_sess.reset();
    g_peer.reset();
    g_finalized = true;
    return MPI_SUCCESS;
}

int MPI_Initialized(int *flag)
{
    *flag = (g_sess || g_finalized) ? 1 : 0;
    return MPI_SUCCESS;
}

int MPI_Finalized(int *flag)
{
    *flag = g_finalized ? 1 : 0;
    return MPI_SUCCESS;
}

int MPI_Abort(MPI_Comm, int errorcode)
{
    // the other ranks learn from the closed connections (peer_failure)
    std::fflush(nullptr);
    std::_Exit(errorcode);
}

int MPI_Get_processor_name(char *name, int *resultlen)
{
    if (::gethostname(name, MPI_MAX_PROCESSOR_NAME) != 0) { std::snprintf(name, MPI_MAX_PROCESSOR_NAME, "localhost"); }
    name[MPI_MAX_PROCESSOR_NAME - 1] = 0;
    *resultlen = static_cast<int>(std::strlen(name));
    return MPI_SUCCESS;
}

double MPI_Wtime(void)
{
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int MPI_Comm_rank(MPI_Comm, int *p)
{
    if (!g_sess) { return MPI_ERR_OTHER; }
    *p = static_cast<int>(g_sess->rank());
    return MPI_SUCCESS;
}

int MPI_Comm_size(MPI_Comm, int *p)
{
    if (!g_sess) { return MPI_ERR_OTHER; }
    *p = static_cast<int>(g_sess->size());
    return MPI_SUCCESS;
}

int MPI_Allreduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype datatype, MPI_Op op,
                  MPI_Comm)
{
    sc::dtype dt;
    sc::reduce_op rop;
    if (count < 0 || !to_dtype(datatype, dt) || !to_op(op, rop)) { return MPI_ERR_OTHER; }
    if (sendbuf == MPI_IN_PLACE) { sendbuf = recvbuf; }
    return guarded([&] { g_sess->all_reduce(sendbuf, recvbuf, static_cast<size_t>(count), dt, rop); });
}

int MPI_Barrier(MPI_Comm)
{
    return guarded([&] { g_sess->barrier(); });
}

int MPI_Bcast(void *buffer, int count, MPI_Datatype datatype, int root, MPI_Comm)
{
    sc::dtype dt;
    if (count < 0 || !to_dtype(datatype, dt) || root < 0) { return MPI_ERR_OTHER; }
    return guarded([&] {
        g_sess->broadcast(buffer, buffer, static_cast<size_t>(count), dt, "", nullptr,
                          static_cast<size_t>(root));
    });
}

int MPI_Allgather(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf,
                  int recvcount, MPI_Datatype recvtype, MPI_Comm)
{
    sc::dtype dt;
    if (sendcount < 0 || sendcount != recvcount || sendtype != recvtype ||
        !to_dtype(sendtype, dt)) {
        return MPI_ERR_OTHER;
    }
    return guarded([&] { g_sess->all_gather(sendbuf, recvbuf, static_cast<size_t>(sendcount), dt); });
}

int MPI_Reduce(const void *sendbuf, void *recvbuf, int count, MPI_Datatype datatype, MPI_Op op,
               int root, MPI_Comm)
{
    sc::dtype dt;
    sc::reduce_op rop;
    if (count < 0 || !to_dtype(datatype, dt) || !to_op(op, rop) || root < 0) {
        return MPI_ERR_OTHER;
    }
    if (sendbuf == MPI_IN_PLACE) { sendbuf = recvbuf; }
    return guarded([&] {
        g_sess->reduce(sendbuf, recvbuf, static_cast<size_t>(count), dt, rop, "", nullptr,
                       static_cast<size_t>(root));
    });
}

int MPI_Gather(const void *sendbuf, int sendcount, MPI_Datatype sendtype, void *recvbuf,
               int recvcount, MPI_Datatype recvtype, int root, MPI_Comm)
{
    sc::dtype dt;
    if (sendcount < 0 || root < 0 || !to_dtype(sendtype, dt)) { return MPI_ERR_OTHER; }
    if (g_sess && g_sess->rank() == static_cast<size_t>(root) &&
        (sendcount != recvcount || sendtype != recvtype)) {
        return MPI_ERR_OTHER;
    }
    return guarded([&] {
        g_sess->gather(sendbuf, recvbuf, static_cast<size_t>(sendcount), dt, "",
                       static_cast<size_t>(root));
    });
}

int MPI_Send(const void *buf, int count, MPI_Datatype datatype, int dest, int tag, MPI_Comm)
{
    sc::dtype dt;
    if (count < 0 || dest < 0 || !to_dtype(datatype, dt)) { return MPI_ERR_OTHER; }
    return guarded([&] {
        g_sess->send(buf, static_cast<size_t>(count), dt, static_cast<size_t>(dest),
                     "mpi/tag/" + std::to_string(tag));
    });
}

int MPI_Recv(void *buf, int count, MPI_Datatype datatype, int source, int tag, MPI_Comm,
             MPI_Status *status)
{
    sc::dtype dt;
    if (count < 0 || source < 0 || !to_dtype(datatype, dt)) { return MPI_ERR_OTHER; }
    const int rc = guarded([&] {
        g_sess->recv(buf, static_cast<size_t>(count), dt, static_cast<size_t>(source),
                     "mpi/tag/" + std::to_string(tag));
    });
    if (status != MPI_STATUS_IGNORE) {
        status->MPI_SOURCE = source;
        status->MPI_TAG = tag;
        status->MPI_ERROR = rc;
    }
    return rc;
}
}
