// Point-to-point: pass a token around the ring of ranks.
#include <cstdio>
#include <thread>

#include <stdml/collective>

using namespace stdml::collective;

int main()
{
    auto p = peer::from_env();
    session sess = p.join();
    const size_t n = sess.size(), r = sess.rank();
    if (n == 1) {
        std::printf("single rank: nothing to pass\n");
        return 0;
    }
    int token = 0;
    if (r == 0) {
        token = 100;
        sess.send(&token, 1, i32, 1, "token");
        sess.recv(&token, 1, i32, n - 1, "token");
        std::printf("token came back as %d (expected %zu)\n", token, 100 + n - 1);
        return token == static_cast<int>(100 + n - 1) ? 0 : 1;
    }
    sess.recv(&token, 1, i32, r - 1, "token");
    ++token;
    sess.send(&token, 1, i32, (r + 1) % n, "token");
    return 0;
}
