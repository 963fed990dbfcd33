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
    printf("rank %d/%d: %s\n", rank, size, bad == 0 ? "OK" : "WRONG");
    MPI_Finalize();
    return bad == 0 ? 0 : 1;
}
