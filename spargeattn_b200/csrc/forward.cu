// One call for the whole path of spas_sage2_attn_meansim_topk_cuda / spas_sage2_attn_meansim_cuda
// (spas_sage_attn/core.py:39-169): K mean, pooling + self-similarity + INT8 quantisation of Q and K, block
// selection + LUT, FP8 quantisation of V, block-sparse attention -- the sequence a host otherwise issues entry by
// entry, here on one stream with every intermediate tensor carved out of one caller-provided workspace. It exists
// for small problems, where issuing the nine launches from an interpreter costs more than running them.
#include "common.cuh"

namespace sparge {

enum { kWsKm, kWsScratch, kWsPq, kWsPk, kWsSimQ, kWsSimK, kWsQ8, kWsK8, kWsQs, kWsKs, kWsLut, kWsValid, kWsV8, kWsVs, kWsCount };

static size_t round_up_256(size_t x) { return (x + 255) / 256 * 256; }

// Offsets of the workspace parts (each 256-byte aligned); returns the total size.
static size_t forward_layout(int B, int H, int N, int D, size_t* off) {
  const size_t BH = (size_t)B * H, nq = ((size_t)N + 127) / 128, nk = ((size_t)N + 63) / 64, npad = nq * 128;
  const size_t bytes[kWsCount] = {
      BH * D * 2,                                  // km
      sparge_k_mean_scratch_bytes(B, H, N, D),     // k-mean partial sums
      BH * nq * D * 2, BH * nk * D * 2,            // pooled q, pooled k
      BH * nq, BH * nk,                            // self-similarity flags
      BH * (size_t)N * D, BH * (size_t)N * D,      // q_int8, k_int8
      BH * nq * 4, BH * nk * 4,                    // q_scale, k_scale
      BH * nq * nk * 4, BH * nq * 4,               // lut, valid
      BH * npad * D, BH * D * 4};                  // v8, v_scale
  size_t total = 0;
  for (int i = 0; i < kWsCount; i++) {
    if (off) off[i] = total;
    total += round_up_256(bytes[i]);
  }
  return total;
}

}  // namespace sparge

extern "C" size_t sparge_forward_workspace_bytes(int B, int H, int N, int D) {
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128)) return 0;
  return sparge::forward_layout(B, H, N, D, nullptr);
}

extern "C" int sparge_forward_workspace_layout(int B, int H, int N, int D, size_t* offsets, int n_offsets) {
  if (!offsets) return SPARGE_ERR_NULL;
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128) || n_offsets != sparge::kWsCount) return SPARGE_ERR_INVALID_ARG;
  sparge::forward_layout(B, H, N, D, offsets);
  return SPARGE_OK;
}

extern "C" int sparge_meansim_forward(const void* q, const void* k, const void* v, void* o, const float* simthreshd1,
                                      const float* cdfthreshd, const float* topk, const float* pvthreshd, void* workspace,
                                      size_t workspace_bytes, int32_t* dev_status, int B, int H, int N, int D, int dtype,
                                      int v_dtype, int is_causal, int kernel_causal, int attention_sink, int smooth_k,
                                      float sm_scale, const long long* q_strides, const long long* k_strides,
                                      const long long* v_strides, const long long* o_strides, sparge_stream_t stream) {
  using namespace sparge;
  if (!q || !k || !v || !o || !simthreshd1 || !workspace || !q_strides || !k_strides || !v_strides || !o_strides)
    return SPARGE_ERR_NULL;
  if ((cdfthreshd == nullptr) == (topk == nullptr)) return SPARGE_ERR_INVALID_ARG;   // exactly one selection rule
  if (B <= 0 || H <= 0 || N < 128 || (D != 64 && D != 128)) return SPARGE_ERR_INVALID_ARG;
  if (reinterpret_cast<uintptr_t>(workspace) & 255) return SPARGE_ERR_INVALID_ARG;
  size_t off[kWsCount];
  if (workspace_bytes < forward_layout(B, H, N, D, off)) return SPARGE_ERR_INVALID_ARG;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  void* km = ws + off[kWsKm];
  const int nq = (N + 127) / 128, nk = (N + 63) / 64;
  int rc = SPARGE_OK;
  if (smooth_k) {
    rc = sparge_k_mean_strided(k, km, ws + off[kWsScratch], B, H, N, D, dtype, k_strides[0], k_strides[1], k_strides[2], stream);
    if (rc != SPARGE_OK) return rc;
  }
  rc = sparge_pool_quant_strided(q, nullptr, simthreshd1, ws + off[kWsPq], ws + off[kWsSimQ], (int8_t*)(ws + off[kWsQ8]),
                                 (float*)(ws + off[kWsQs]), B, H, N, D, 128, dtype, q_strides[0], q_strides[1], q_strides[2],
                                 stream);
  if (rc != SPARGE_OK) return rc;
  rc = sparge_pool_quant_strided(k, smooth_k ? km : nullptr, simthreshd1, ws + off[kWsPk], ws + off[kWsSimK],
                                 (int8_t*)(ws + off[kWsK8]), (float*)(ws + off[kWsKs]), B, H, N, D, 64, dtype, k_strides[0],
                                 k_strides[1], k_strides[2], stream);
  if (rc != SPARGE_OK) return rc;
  // the skip test exempts the last two live blocks of the visiting order: best-first order only without it
  rc = sparge_select(ws + off[kWsPq], ws + off[kWsPk], ws + off[kWsSimQ], ws + off[kWsSimK], topk, cdfthreshd, nullptr,
                     (int32_t*)(ws + off[kWsLut]), (int32_t*)(ws + off[kWsValid]), B, H, nq, nk, D, dtype, is_causal,
                     attention_sink, pvthreshd ? SPARGE_LUT_ASCENDING : SPARGE_LUT_BEST_FIRST, stream);
  if (rc != SPARGE_OK) return rc;
  rc = sparge_quant_v_strided(v, ws + off[kWsV8], (float*)(ws + off[kWsVs]), B, H, N, D, v_dtype, v_strides[0], v_strides[1],
                              v_strides[2], stream);
  if (rc != SPARGE_OK) return rc;
  return sparge_attn_fwd_strided((const int8_t*)(ws + off[kWsQ8]), (const int8_t*)(ws + off[kWsK8]), ws + off[kWsV8], o,
                                 (const int32_t*)(ws + off[kWsLut]), (const int32_t*)(ws + off[kWsValid]), pvthreshd,
                                 (const float*)(ws + off[kWsQs]), (const float*)(ws + off[kWsKs]),
                                 (const float*)(ws + off[kWsVs]), dev_status, B, H, N, D, dtype, kernel_causal, sm_scale,
                                 o_strides[0], o_strides[1], o_strides[2], stream);
}
