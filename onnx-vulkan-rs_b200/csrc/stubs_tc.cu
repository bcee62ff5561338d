// Placeholders until the tensor-core kernels are in: nothing applies, so the
// general kernels run.
#include "ovk_internal.h"
#include "epilogue.cuh"
struct ConvGeom;
bool ovk_nbits_gemm_applies(const ovk_ctx *, const ovk_nbits_weight *, int64_t, int32_t, int32_t, const void *, const void *) { return false; }
int32_t ovk_nbits_gemm(ovk_ctx *ctx, const ovk_nbits_weight *, const void *, int32_t, int64_t, void *, int32_t) { return ovk_fail(ctx, OVK_UNSUPPORTED, "nbits gemm kernel not built"); }
bool ovk_qconv_tc_applies(const ovk_ctx *, const ovk_qconv_weight *, const ConvGeom &, const void *) { return false; }
int32_t ovk_qconv_tc_launch(ovk_ctx *ctx, const ovk_qconv_weight *, const void *, int32_t, const ConvGeom &, int32_t, int32_t, const EpiParams &, void *) { return ovk_fail(ctx, OVK_UNSUPPORTED, "qconv tc kernel not built"); }
int32_t ovk_qconv_tc_prepare_weight(ovk_ctx *, ovk_qconv_weight *) { return OVK_OK; }
