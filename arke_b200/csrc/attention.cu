#include "capi_internal.h"
using namespace arke;
extern "C" int arke_b200_gqa_fwd(const void*, const void*, const void*, void*, float*, int, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int, float, void*) { return set_error(ARKE_ERR_ARG, "gqa_fwd: not built"); }
