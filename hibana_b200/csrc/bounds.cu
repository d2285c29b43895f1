// Host side of the checked-index build flavour (see `index_ok` in hb_common.cuh). The normal build only answers
// that it has no checks; the flavour built with -DHB_BOUNDS -rdc=true holds the limit table and the first
// violation's record. The reference has no counterpart: it relies on compute-sanitizer runs.
#include "hb_api.h"
#include "hb_common.cuh"

#ifdef HB_BOUNDS
namespace hb {
__device__ BoundsState g_bounds;
}
#endif

extern "C" {

int hb_bounds_enabled() {
#ifdef HB_BOUNDS
  return 1;
#else
  return 0;
#endif
}

// which: 0 KV slots, 1 recurrent-state slots, 2 vocabulary, 3 block-table rows. value <= 0 switches the check off.
int hb_bounds_set(int which, long long value) {
#ifdef HB_BOUNDS
  if (which < 0 || which >= hb::kBoundKinds) return 1;
  return cudaMemcpyToSymbol(hb::g_bounds, &value, sizeof(value), offsetof(hb::BoundsState, limit) + which * sizeof(long long)) ==
                 cudaSuccess
             ? 0
             : 2;
#else
  (void)which;
  (void)value;
  return 0;
#endif
}

// out[4] = {violations so far, kernel of the first, its index, the limit it broke}; clears the record.
int hb_bounds_read(long long* out) {
#ifdef HB_BOUNDS
  hb::BoundsState st;
  if (cudaMemcpyFromSymbol(&st, hb::g_bounds, sizeof(st)) != cudaSuccess) return 2;
  out[0] = st.hits;
  out[1] = st.kernel;
  out[2] = st.index;
  out[3] = st.bound;
  const int zero[2] = {0, 0};
  return cudaMemcpyToSymbol(hb::g_bounds, zero, sizeof(zero), offsetof(hb::BoundsState, hits)) == cudaSuccess ? 0 : 2;
#else
  out[0] = out[1] = out[2] = out[3] = 0;
  return 0;
#endif
}

}  // extern "C"
