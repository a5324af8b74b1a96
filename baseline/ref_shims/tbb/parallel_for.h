// Stand-in for <tbb/parallel_for.h>: see tbb_min.h.
#pragma once
#include "tbb_min.h"
