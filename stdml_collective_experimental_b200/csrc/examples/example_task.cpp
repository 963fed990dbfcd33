// Polled task trees: two sequences run side by side.
#include <stdml/bits/collective/log.hpp>
#include <stdml/bits/collective/task.hpp>

using namespace stdml::collective;

static task *say(const std::string &msg)
{
    return new simple_task([msg] { log(PRINT) << msg; });
}

static task *two_steps(const std::string &a, const std::string &b)
{
    task_builder b2;
    b2 << say(a);
    b2 << say(b);
    return b2.seq();
}

int main()
{
    task_builder all;
    all << two_steps("11", "12");
    all << two_steps("21", "22");
    task *t = all.par();
    t->finish();
    delete t;
    return 0;
}
