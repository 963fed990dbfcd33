// Smallest program: join, all-reduce a vector, print.  Run with
//   stdml_collective_run -np 4 example_1        or        example_1   (single)
#include <iostream>
#include <numeric>
#include <vector>

#include <stdml/collective>

int main()
{
    auto peer = stdml::collective::peer::from_env();
    stdml::collective::session sess = peer.join();
    std::vector<int> x(8), y(8);
    std::iota(x.begin(), x.end(), static_cast<int>(sess.rank()));
    sess.all_reduce(x.data(), x.data() + x.size(), y.data());
    if (sess.rank() == 0) {
        std::cout << "np=" << sess.size() << " sum:";
        for (int v : y) { std::cout << " " << v; }
        std::cout << std::endl;
    }
    return 0;
}
