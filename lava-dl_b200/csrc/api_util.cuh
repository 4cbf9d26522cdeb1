// Argument checking helpers shared by the entry-point translation units.
#pragma once

#include "common.cuh"
#include "ops.cuh"

namespace sb {

int check_geom(const sb_geom* g, RowGeom* out, int64_t n_max);
int check_count(int64_t n, const char* name);
Scale make_scale(int w_scale);

}  // namespace sb

#define SB_TRY(expr)                \
  do {                              \
    int rc__ = (expr);              \
    if (rc__ != SB_OK) return rc__; \
  } while (0)
