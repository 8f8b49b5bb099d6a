// The C++ interface lives with the public headers: include/cuvs/neighbors/ivf_pq.hpp.
#pragma once
#include <cuvs/neighbors/ivf_pq.hpp>
