/* The MPI-shaped C interface: compile as C, link the library.  Run with
 * OMPI_COMM_WORLD_SIZE / OMPI_COMM_WORLD_RANK set (or under stdml_collective_run). */
#include <stdio.h>

#include <stdml/mpi.h>

int main(int argc, char *argv[])
{
    int rank = 0, size = 0, i, bad = 0;
    float x[16], y[16];
    int lo = 0;
    MPI_Init(&argc, &argv);
    MPI_Comm_rank(MPI_COMM_WORLD, &rank);
    MPI_Comm_size(MPI_COMM_WORLD, &size);
    for (i = 0; i < 16; ++i) { x[i] = (float)(rank + i); }
    MPI_Allreduce(x, y, 16, MPI_FLOAT, MPI_SUM, MPI_COMM_WORLD);
    for (i = 0; i < 16; ++i) { bad += y[i] != (float)(size * (size - 1) / 2 + size * i); }
    MPI_Allreduce(&rank, &lo, 1, MPI_INT, MPI_MIN, MPI_COMM_WORLD);
    bad += lo != 0;
    MPI_Barrier(MPI_COMM_WORLD);
    {
        /* beyond the reference's five calls: in place, any broadcast root, gather, send / recv */
        int flag = 0, len = 0, token = -1, last = size - 1, from_last = -1;
        int all[64];
        char host[MPI_MAX_PROCESSOR_NAME];
        double t0 = MPI_Wtime();
        MPI_Status st;
        MPI_Initialized(&flag);
        bad += flag != 1;
        for (i = 0; i < 16; ++i) { y[i] = (float)rank; }
        MPI_Allreduce(MPI_IN_PLACE, y, 16, MPI_FLOAT, MPI_MAX, MPI_COMM_WORLD);
        bad += y[7] != (float)last;
        from_last = rank == last ? 77 : -1;
        MPI_Bcast(&from_last, 1, MPI_INT, last, MPI_COMM_WORLD);
        bad += from_last != 77;
        if (size <= 64) {
            MPI_Gather(&rank, 1, MPI_INT, all, 1, MPI_INT, 0, MPI_COMM_WORLD);
            if (rank == 0) {
                for (i = 0; i < size; ++i) { bad += all[i] != i; }
            }
        }
        if (size > 1) {
            if (rank == 0) {
                token = 4242;
                MPI_Send(&token, 1, MPI_INT, last, 9, MPI_COMM_WORLD);
            } else if (rank == last) {
                MPI_Recv(&token, 1, MPI_INT, 0, 9, MPI_COMM_WORLD, &st);
                bad += token != 4242 || st.MPI_SOURCE != 0 || st.MPI_TAG != 9;
            }
        }
        MPI_Get_processor_name(host, &len);
        bad += len <= 0 || MPI_Wtime() < t0;
        MPI_Barrier(MPI_COMM_WORLD);
    }
    printf("rank %d/%d: %s\n", rank, size, bad == 0 ? "OK" : "WRONG");
    MPI_Finalize();
    {
        int done = 0;
        MPI_Finalized(&done);
        bad += done != 1;
    }
    return bad == 0 ? 0 : 1;
}
