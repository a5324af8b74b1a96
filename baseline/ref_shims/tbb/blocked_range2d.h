// Stand-in for <tbb/blocked_range2d.h>: see tbb_min.h.
#pragma once
#include "tbb_min.h"
