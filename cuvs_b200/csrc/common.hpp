// Shared host-side plumbing lives with the public headers: include/cuvs/core/b200_common.hpp.
#pragma once
#include <cuvs/core/b200_common.hpp>
