// Stand-in for <tbb/info.h>: see tbb_min.h.
#pragma once
#include "tbb_min.h"
