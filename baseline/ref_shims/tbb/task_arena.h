// Stand-in for <tbb/task_arena.h>: see tbb_min.h.
#pragma once
#include "tbb_min.h"
