// Stand-in for <tbb/scalable_allocator.h>: see tbb_min.h.
#pragma once
#include "tbb_min.h"
