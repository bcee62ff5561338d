// Placeholders until the tensor-core kernels are in: nothing applies, so the
// general kernels run.
#include "ovk_internal.h"
#include "epilogue.cuh"
struct ConvGeom;
bool ovk_qconv_tc_applies(const ovk_ctx *, const ovk_qconv_weight *, const ConvGeom &, const void *) { return false; }
int32_t ovk_qconv_tc_launch(ovk_ctx *ctx, const ovk_qconv_weight *, const void *, int32_t, const ConvGeom &, int32_t, int32_t, const EpiParams &, void *) { return ovk_fail(ctx, OVK_UNSUPPORTED, "qconv tc kernel not built"); }
int32_t ovk_qconv_tc_prepare_weight(ovk_ctx *, ovk_qconv_weight *) { return OVK_OK; }
