// Free-function spelling of the collectives over a default session, for code
// that does not want to carry peer/session objects around.  The reference
// declares these names without defining most of them
// (include/stdml/bits/collective/algorithm.hpp:6-18); here they are all live.
#pragma once
#include <cstddef>

#include <stdml/bits/collective/dtype.hpp>
#include <stdml/bits/collective/elastic.hpp>

namespace stdml::collective
{
class session;

// creates the default peer from the environment and joins; idempotent
void init();
void finalize();
session &default_session();
resize_result resize(size_t new_size);

void all_reduce(const void *input, void *output, size_t count, dtype dt, reduce_op op = sum);
void reduce(const void *input, void *output, size_t count, dtype dt, reduce_op op = sum);
void all_gather(const void *input, void *output, size_t count, dtype dt);
void gather(const void *input, void *output, size_t count, dtype dt);
void broadcast(const void *input, void *output, size_t count, dtype dt);
}  // namespace stdml::collective
