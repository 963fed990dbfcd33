// prun(): fork the ranks from one program, no launcher needed.
#include <cstdio>

#include <stdml/collective>

int main(int argc, char *argv[])
{
    const int np = argc > 1 ? std::atoi(argv[1]) : 4;
    stdml::collective::prun(np, [](stdml::collective::session &sess) {
        const int total = sess.all_reduce(static_cast<int>(sess.rank()) + 1);
        std::printf("rank %zu of %zu: total %d\n", sess.rank(), sess.size(), total);
    });
    return 0;
}
