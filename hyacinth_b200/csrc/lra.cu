// placeholder: fitting drivers follow
#include "hyb_internal.h"
extern "C" int32_t hyacinInterpolateFit(const hyacinHandle_t*, double, char, int32_t, int32_t, int32_t, const void*, int32_t, int32_t*, void*, int32_t, int64_t, hyacinPrecision_t) { return 0; }
extern "C" int32_t hyacinTsvdFit(const hyacinHandle_t*, double, char, int32_t, int32_t, int32_t, const void*, int32_t, void*, void*, int32_t, int64_t, hyacinPrecision_t) { return 0; }
extern "C" int32_t hyacinTsvdFitSegmentN(const hyacinHandle_t*, double, char, int32_t, int32_t, int32_t, const void*, int32_t, void*, void*, int32_t, int64_t, hyacinPrecision_t) { return 0; }
extern "C" int32_t hyacinXGevd(const hyacinHandle_t*, double, int32_t, int32_t, hyacinPrecision_t, void*, int32_t, void*, hyacinPrecision_t, void*, int32_t) { return 0; }
extern "C" int32_t hyacinXGinterp(const hyacinHandle_t*, double, int32_t, int32_t, hyacinPrecision_t, void*, int32_t, int32_t*, hyacinPrecision_t, void*, int32_t) { return 0; }
extern "C" double hyacinCheckNorm(const hyacinHandle_t*, char, int32_t, int32_t, const void*, int32_t, int32_t, const void*, int32_t, hyacinPrecision_t) { return 0.; }
