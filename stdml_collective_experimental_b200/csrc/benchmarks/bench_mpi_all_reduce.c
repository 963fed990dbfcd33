/* The reference's MPI micro-benchmark shape (benchmarks/bench-mpi-all-reduce.c:110-120:
 * 100 tensors of 1024 floats, 10 steps) through the MPI facade. */
#include <stdio.h>
#include <stdlib.h>
#include <time.h>

#include <stdml/mpi.h>

static double now(void)
{
    struct timespec ts;
    clock_gettime(CLOCK_MONOTONIC, &ts);
    return ts.tv_sec + ts.tv_nsec * 1e-9;
}

int main(int argc, char *argv[])
{
    const int tensors = argc > 1 ? atoi(argv[1]) : 100;
    const int count = argc > 2 ? atoi(argv[2]) : 1024;
    const int steps = argc > 3 ? atoi(argv[3]) : 10;
    int rank, size, i, s;
    float *x = (float *)malloc(sizeof(float) * count), *y = (float *)malloc(sizeof(float) * count);
    MPI_Init(&argc, &argv);
    MPI_Comm_rank(MPI_COMM_WORLD, &rank);
    MPI_Comm_size(MPI_COMM_WORLD, &size);
    for (i = 0; i < count; ++i) { x[i] = 1.0f; }
    for (s = 0; s < steps; ++s) {
        const double t0 = now();
        for (i = 0; i < tensors; ++i) { MPI_Allreduce(x, y, count, MPI_FLOAT, MPI_SUM, MPI_COMM_WORLD); }
        {
            const double d = now() - t0;
            const double gibs = 4.0 * (size - 1) * tensors * count * 4.0 / d / 1073741824.0;
            if (rank == 0) { printf("step %d %.3f GiB/s | %.3f ms\n", s + 1, gibs, d * 1e3); }
        }
    }
    if (y[0] != (float)size) {
        printf("WRONG result %f\n", y[0]);
        return 1;
    }
    MPI_Finalize();
    free(x);
    free(y);
    return 0;
}
