// Host entry points of the checked build (see the "checked build" block in common.cuh).  In a release build they
// report that checking is off and do nothing else.
#include "common.cuh"

using namespace poot;

POOT_API int poot_debug_bounds_enabled() {
#ifdef POOT_DEBUG_BOUNDS
  return 1;
#else
  return 0;
#endif
}

// out4 = {site, source line, index, bound} of the first recorded fault over all translation units, zeros when there is
// none.  Synchronises the device (it is read after a step, never inside one).
POOT_API int poot_debug_bounds_read(int* out4) {
  out4[0] = out4[1] = out4[2] = out4[3] = 0;
#ifdef POOT_DEBUG_BOUNDS
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  for (const dbg::Unit& u : dbg::units()) {
    int f[4];
    int rc = u.read(f);
    if (rc != 0) return rc;
    if (f[0] != 0) {
      for (int i = 0; i < 4; ++i) out4[i] = f[i];
      return 0;
    }
  }
#endif
  return 0;
}

POOT_API int poot_debug_bounds_clear() {
#ifdef POOT_DEBUG_BOUNDS
  for (const dbg::Unit& u : dbg::units()) {
    int rc = u.clear();
    if (rc != 0) return rc;
  }
#endif
  return 0;
}

// which: 0 pool slots, 1 pool blocks, 2 recurrent-state rows; value <= 0 means unknown (checks against it pass).
POOT_API int poot_debug_bounds_limit(int which, long long value) {
  if (which < 0 || which >= kLimCount) return (int)cudaErrorInvalidValue;
#ifdef POOT_DEBUG_BOUNDS
  for (const dbg::Unit& u : dbg::units()) {
    int rc = u.limit(which, value);
    if (rc != 0) return rc;
  }
#endif
  return 0;
}

POOT_API int poot_debug_bounds_units() {
#ifdef POOT_DEBUG_BOUNDS
  return (int)dbg::units().size();
#else
  return 0;
#endif
}
