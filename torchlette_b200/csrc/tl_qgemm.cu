// Prefill GEMM with fused dequantization (tcgen05 / TMEM) — placeholder until the kernel lands.
#include "tl_common.cuh"

bool tl_qgemm_variant_applicable(const tl_variant& v, int64_t m, int64_t n, int64_t k, int32_t a_dtype,
                                 const tl_quant_desc& q) {
  (void)v; (void)m; (void)n; (void)k; (void)a_dtype; (void)q;
  return false;
}
int32_t tl_qgemm_default_variant(tl_ctx* ctx, int64_t, int64_t, int64_t, int32_t, const tl_quant_desc&, tl_variant* out) {
  (void)ctx;
  *out = tl_variant{TL_FAMILY_QGEMM, 0, 0, 0, 0, 0};
  return TL_OK;
}
int32_t tl_qgemm_candidates(tl_ctx*, int64_t, int64_t, int64_t, int32_t, const tl_quant_desc&, std::vector<tl_variant>* out) {
  out->clear();
  return TL_OK;
}
int32_t tl_launch_qgemm(tl_ctx* ctx, const tl_variant&, const void*, int32_t, const void*, const void*, void*, int32_t,
                        int64_t, int64_t, int64_t, const tl_quant_desc&, const EpiParams&, tl_plan_receipt*) {
  return tl_set_error(ctx, TL_ERR_UNIMPLEMENTED, "tl_qgemm_nt: not implemented yet");
}
