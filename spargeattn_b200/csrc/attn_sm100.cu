// LUT-driven block-sparse attention for sm_100a.
//   S = Q8 K8^T   : tcgen05.mma kind::i8, operands staged by TMA into 128B/64B-swizzled smem,
//                   s32 accumulator in tensor memory (TMEM). Two live 64-key blocks are paired into one
//                   N = 128 step: their K tiles sit next to each other in shared memory, so one
//                   instruction covers both (an odd last block runs as N = 64).
//   online softmax in registers, two threads per query row (one per block of the pair; they exchange their
//                   row maxima through shared memory): one running-maximum update, one output rescale and
//                   one round of hand-offs per 128 keys; P rounded to e4m3 and stored to a 128B-swizzled
//                   shared-memory tile
//   O += P8 V8    : tcgen05.mma kind::f8f6f4, A = P tile (K-major), B = V tiles (token-major,
//                   MN-major descriptor), f32 accumulator in TMEM
// Replaces qk_int_sv_f8_block_sparse_attn_kernel (csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:42-755)
// and its host wrapper (csrc/qattn/qk_int_sv_f8_cuda_sm89.cu:392-585).
//
// One CTA per (q-block of 128 rows, head, batch); 10 warps:
//   warps 0-7  softmax / correction / epilogue (warps w and w + 4 own query rows 32 (w & 3) ... = TMEM lanes)
//   warp  8    TMA producer: walks the delta-encoded LUT and fetches only live K/V blocks
//   warp  9    MMA issuer (one elected lane) and TMEM owner
// Sixteen softmax warps per SM (two CTAs): four per scheduler, enough to keep the exponential unit fed while
// other warps wait on a hand-off.
// TMEM columns: [0,128) S of the current step, [128,128+D) O  -> 256 columns, two CTAs per SM.
// S is single-buffered: the softmax warps release it as soon as their last tcgen05.ld of the step has
// landed (half way through the step), and QK^T of the next step runs under the second half's exponentials.
//
// Every wait is bounded; on expiry the kernel records a code in *dev_status and unwinds.
#include <cuda.h>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace sparge {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kFp8Offset = 8.807f;     // csrc/qattn/attn_utils.cuh:28-30: 2^8.807 = 448 = e4m3 max
constexpr float kMaskValue = -5000000.0f;  // csrc/qattn/attn_utils.cuh:348-352
constexpr uint32_t kMagicBits = 0x4B400000u;   // bit pattern of 12582912.0f = 1.5 * 2^23
constexpr float kMagic = 12582912.0f;
constexpr float kFastScaleLimit = 0.0078125f;  // 2^-7: bounds the fast path's per-block weight error by 0.41 %


// PVF16: P and V in fp16 (tcgen05.mma kind::f16) instead of e4m3 -- the arithmetic of the reference's fp16-PV kernel
// (csrc/qattn/qk_int_sv_f16_cuda_sm80.cuh), which its Sage1-signature entry points run. V then is the caller's fp16
// tensor itself (no quantiser); a 64-key V tile is D/64 sub-tiles of [64 keys x 128 bytes] (64 channels each, 128B
// swizzle), P is two sub-tiles of [128 rows x 128 bytes], one per block of a pair. The tiles are twice as large,
// so the rings are shorter (see kKTiles) to keep two CTAs per SM.
template <int D, bool PVF16 = false>
struct AttnShape {
  // K ring of single tiles (fp16 variant at D = 128): three 64-key tile slots instead of two pair slots, and one V
  // pair slot, bring the CTA down to 105 KB of shared memory so that two fit per SM; a step's two K tiles are then not
  // adjacent and QK^T is issued as two N = 64 instruction groups.
  static constexpr bool kKTiles = PVF16 && D == 128;
  static constexpr int kStagesK = kKTiles ? 3 : (D == 128 || PVF16) ? 2 : 4;   // ring slots: PAIRS of 64-key tiles (tiles if kKTiles)
  static constexpr int kStagesV = kKTiles ? 1 : (D == 128 || PVF16) ? 2 : 4;
  static constexpr int kTileQ = 128 * D;
  static constexpr int kTileKV = 64 * D;
  static constexpr int kPairKV = 2 * kTileKV;
  static constexpr int kTileV = PVF16 ? 2 * kTileKV : kTileKV;
  static constexpr int kPairV = 2 * kTileV;
  static constexpr int kTileP = PVF16 ? 2 * 128 * 128 : 128 * 128;   // 128 rows x 128 keys of e4m3 / fp16
  static constexpr int kRingK = kStagesK * (kKTiles ? kTileKV : kPairKV);
  static constexpr int kSmemBytes = 1024 + kTileQ + kTileP + kRingK + kStagesV * kPairV;
  static constexpr int kTmemCols = 256;
  static constexpr int kCtasPerSm = 2;
  static constexpr uint32_t kSwizzle = (D == 128) ? kSwizzle128B : kSwizzle64B;
};

__device__ __forceinline__ void report(int32_t* status, int code) {
  if (status) atomicCAS(status, 0, code);
}

template <typename OutT>
__device__ __forceinline__ uint32_t pack2(float a, float b);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void st_shared_v4(uint32_t addr, const uint32_t* w) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]) : "memory");
}

// Row maximum of 32 scores, in log2 units. klim: keys with local index >= klim are masked.
template <bool MASKED>
__device__ __forceinline__ float chunk_rowmax(const uint32_t* sr, float c, int klim) {
  if (!MASKED) {
    int m0 = (int)sr[0], m1 = (int)sr[8], m2 = (int)sr[16], m3 = (int)sr[24];   // four chains: short latency
#pragma unroll
    for (int k = 1; k < 7; k += 2) {
      m0 = __vimax3_s32(m0, (int)sr[k], (int)sr[k + 1]);
      m1 = __vimax3_s32(m1, (int)sr[8 + k], (int)sr[8 + k + 1]);
      m2 = __vimax3_s32(m2, (int)sr[16 + k], (int)sr[16 + k + 1]);
      m3 = __vimax3_s32(m3, (int)sr[24 + k], (int)sr[24 + k + 1]);
    }
    m0 = __vimax3_s32(m0, m1, (int)sr[7]);
    m2 = __vimax3_s32(m2, m3, (int)sr[15]);
    const int mx = max(__vimax3_s32(m0, m2, (int)sr[23]), (int)sr[31]);
    return (__int_as_float(mx + (int)kMagicBits) - kMagic) * c;   // c > 0: max commutes with the scaling
  } else {
    int mx = INT_MIN;
#pragma unroll
    for (int k = 0; k < 32; k++) mx = (k < klim) ? max(mx, (int)sr[k]) : mx;
    return (klim > 0) ? __int2float_rn(mx) * c : kMaskValue;
  }
}

// Per-thread granularity (QuantGranularity::kPerThread, qk_int_sv_f8_cuda_sm89.cuh:116-136): key column n of a
// block is scaled by entry (n % 8) / 2 of the block's four K scales, so a thread's 32 scores carry four different
// factors c4[0..3] and the integer maximum no longer commutes with the scaling: one maximum per factor.
__device__ __forceinline__ float chunk_rowmax_g(const uint32_t* sr, const float* c4, int klim) {
  int mx[4] = {INT_MIN, INT_MIN, INT_MIN, INT_MIN};
#pragma unroll
  for (int k = 0; k < 32; k++) mx[(k & 7) >> 1] = (k < klim) ? max(mx[(k & 7) >> 1], (int)sr[k]) : mx[(k & 7) >> 1];
  float r = kMaskValue;
#pragma unroll
  for (int g = 0; g < 4; g++) r = (mx[g] != INT_MIN) ? fmaxf(r, __int2float_rn(mx[g]) * c4[g]) : r;
  return r;
}

__device__ __forceinline__ float chunk_exp_g(const uint32_t* sr, const float* c4, float m, int klim, uint32_t prow,
                                             int chunk0, int rsw) {
  uint32_t pr[4];
  const float off = kFp8Offset - m;
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < 32; k += 4) {
    float p0 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 0]), c4[((k + 0) & 7) >> 1], off));
    float p1 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 1]), c4[((k + 1) & 7) >> 1], off));
    float p2 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 2]), c4[((k + 2) & 7) >> 1], off));
    float p3 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 3]), c4[((k + 3) & 7) >> 1], off));
    p0 = (k + 0 < klim) ? p0 : 0.f;
    p1 = (k + 1 < klim) ? p1 : 0.f;
    p2 = (k + 2 < klim) ? p2 : 0.f;
    p3 = (k + 3 < klim) ? p3 : 0.f;
    sum += (p0 + p1) + (p2 + p3);
    pr[(k >> 2) & 3] = cvt_e4m3x4(p0, p1, p2, p3);
    if ((k & 12) == 12) st_shared_v4(prow + (uint32_t)(((chunk0 + (k >> 4)) ^ rsw) << 4), pr);
  }
  return sum;
}

// P = 2^(S*c - m + 8.807) for 32 scores: row sum in fp32 before the e4m3 rounding
// (ComputeUnit::kCudaCore, qk_int_sv_f8_cuda_sm89.cuh:773), bytes stored to the row's two 16-byte chunks
// chunk0, chunk0+1 of the 128B-swizzled P tile. `prow` = shared address of the row, rsw = row & 7.
template <bool EXACT>
__device__ __forceinline__ float chunk_exp(const uint32_t* sr, float c, float m, int klim, int one, uint32_t prow,
                                           int chunk0, int rsw) {
  uint32_t pr[4];
  if (!EXACT) {
    // int32 -> fp32 by adding the bit pattern of 1.5 * 2^23 (exact for |S| < 2^22; here |S| <= 127^2 * 128);
    // the 2^23 bias is taken out again inside the FMA constant. Packed f32x2 FMA / ADD halve the issue slots.
    // That constant is rounded at the magnitude of 1.5 * 2^23 * c, so the exponents of this block are off
    // by a common amount of at most 0.75 * c: blocks whose scale is not small take the exact path.
    // `one` is a kernel argument equal to 1 that the compiler cannot fold: multiplying by it turns the
    // int->float bias add into an IMAD, which issues on the FMA pipe instead of the half-rate integer pipe.
    // (Pre-loading the accumulator with the bias through tcgen05.cp, so that no add is needed at all, was
    // measured 14 % slower: the sixteen 4 KB copies per step delay QK^T more than 64 IMADs cost. Evaluating
    // a quarter or half of the exponentials as a polynomial on the FMA pipe was 1.5 - 12 % slower: the loop
    // is bound by issue slots, and each such element costs four more of them than a MUFU does.)
    const float off = fmaf(-kMagic, c, kFp8Offset - m);
    const float2 c2 = make_float2(c, c), o2 = make_float2(off, off);
    float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 32; k += 4) {
      float2 a = make_float2(__int_as_float((int)sr[k + 0] * one + (int)kMagicBits),
                             __int_as_float((int)sr[k + 1] * one + (int)kMagicBits));
      float2 bb = make_float2(__int_as_float((int)sr[k + 2] * one + (int)kMagicBits),
                              __int_as_float((int)sr[k + 3] * one + (int)kMagicBits));
      a = __ffma2_rn(a, c2, o2);
      bb = __ffma2_rn(bb, c2, o2);
      a.x = ex2_approx(a.x);
      a.y = ex2_approx(a.y);
      bb.x = ex2_approx(bb.x);
      bb.y = ex2_approx(bb.y);
      s0 = __fadd2_rn(s0, a);
      s1 = __fadd2_rn(s1, bb);
      pr[(k >> 2) & 3] = cvt_e4m3x4(a.x, a.y, bb.x, bb.y);
      if ((k & 12) == 12) st_shared_v4(prow + (uint32_t)(((chunk0 + (k >> 4)) ^ rsw) << 4), pr);
    }
    s0 = __fadd2_rn(s0, s1);
    return s0.x + s0.y;
  } else {
    const float off = kFp8Offset - m;
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < 32; k += 4) {
      float p0 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 0]), c, off));
      float p1 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 1]), c, off));
      float p2 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 2]), c, off));
      float p3 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 3]), c, off));
      p0 = (k + 0 < klim) ? p0 : 0.f;
      p1 = (k + 1 < klim) ? p1 : 0.f;
      p2 = (k + 2 < klim) ? p2 : 0.f;
      p3 = (k + 3 < klim) ? p3 : 0.f;
      sum += (p0 + p1) + (p2 + p3);
      pr[(k >> 2) & 3] = cvt_e4m3x4(p0, p1, p2, p3);
      if ((k & 12) == 12) st_shared_v4(prow + (uint32_t)(((chunk0 + (k >> 4)) ^ rsw) << 4), pr);
    }
    return sum;
  }
}

// PVF16: P = 2^(S*c - m) for 32 scores as fp16 (no offset: the values are at most 1), row sum in fp32 before the
// rounding; written to the four 16-byte chunks chunk0 .. chunk0+3 of the row in a [128 x 128 B] swizzled sub-tile.
template <bool EXACT>
__device__ __forceinline__ float chunk_exp_f16(const uint32_t* sr, float c, float m, int klim, int one, uint32_t prow,
                                               int chunk0, int rsw) {
  uint32_t pr[4];
  if (!EXACT) {   // same int->float bias trick and packed arithmetic as the e4m3 path (see chunk_exp)
    const float off = fmaf(-kMagic, c, -m);
    const float2 c2 = make_float2(c, c), o2 = make_float2(off, off);
    float2 s0 = make_float2(0.f, 0.f);
#pragma unroll
    for (int k = 0; k < 32; k += 2) {
      float2 a = make_float2(__int_as_float((int)sr[k + 0] * one + (int)kMagicBits),
                             __int_as_float((int)sr[k + 1] * one + (int)kMagicBits));
      a = __ffma2_rn(a, c2, o2);
      a.x = ex2_approx(a.x);
      a.y = ex2_approx(a.y);
      s0 = __fadd2_rn(s0, a);
      const __half2 h = __floats2half2_rn(a.x, a.y);
      pr[(k >> 1) & 3] = *reinterpret_cast<const uint32_t*>(&h);
      if ((k & 6) == 6) st_shared_v4(prow + (uint32_t)(((chunk0 + (k >> 3)) ^ rsw) << 4), pr);
    }
    return s0.x + s0.y;
  }
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < 32; k += 2) {
    float p0 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 0]), c, -m));
    float p1 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 1]), c, -m));
    p0 = (k + 0 < klim) ? p0 : 0.f;
    p1 = (k + 1 < klim) ? p1 : 0.f;
    sum += p0 + p1;
    const __half2 h = __floats2half2_rn(p0, p1);
    pr[(k >> 1) & 3] = *reinterpret_cast<const uint32_t*>(&h);
    if ((k & 6) == 6) st_shared_v4(prow + (uint32_t)(((chunk0 + (k >> 3)) ^ rsw) << 4), pr);
  }
  return sum;
}

__device__ __forceinline__ void pair_sync(int id) {   // the two warps that share 32 query rows
  asm volatile("bar.sync %0, 64;" ::"r"(id) : "memory");
}

constexpr int kAttnThreads = 320;

// GRAN = qk_quant_gran: 1 one Q scale per 128-row block, 2 one per 32-row group (the K scale is per 64-key block in
// both), 3 per-thread Q/K scales. PV_MODE = PVThresholdMode: 0 no skip test, 1 the test decides per block, 2 per
// 32-row group.
template <int D, bool CAUSAL, int PV_MODE, typename OutT, int GRAN, bool PVF16 = false>
__global__ void __launch_bounds__(kAttnThreads, (AttnShape<D, PVF16>::kCtasPerSm))
attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
            const __grid_constant__ CUtensorMap tmap_v, OutT* __restrict__ o, const int32_t* __restrict__ lut,
            const int32_t* __restrict__ valid, const float* __restrict__ pvthr, const float* __restrict__ q_scale,
            const float* __restrict__ k_scale, const float* __restrict__ v_scale, int32_t* dev_status, int N, int H,
            int nq, int nk, float sm_scale_log2, int one, long long osb, long long osh, long long osn,
            int32_t* __restrict__ pv_count, const int32_t* __restrict__ q_ranges) {
  using Shape = AttnShape<D, PVF16>;
  constexpr bool PV_SKIP = PV_MODE != 0, pv_per_warp = PV_MODE == 2, GRAN3 = GRAN == 3;
  constexpr int SK = Shape::kStagesK, SV = Shape::kStagesV;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sP = smem + Shape::kTileQ;
  uint8_t* sK = sP + Shape::kTileP;                  // slot s: sK + s * kPairKV
  uint8_t* sV = sK + Shape::kRingK;                    // slot s: sV + s * kPairV
  constexpr bool KT = Shape::kKTiles;

  __shared__ uint64_t bar_q, bar_k_full[SK], bar_k_empty[SK], bar_v_full[SV], bar_v_empty[SV], bar_s_full, bar_s_free,
      bar_p_ready, bar_o_done, bar_delta[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_skip[2];
  __shared__ float s_delta[2][2][4];   // [step parity][block of the pair][row quarter]
  __shared__ float s_rmax[2][2][128];  // [step parity][thread of the row pair][row]
  __shared__ int4 s_meta[8];           // per step (ring of 8): block indices of the pair and their K scales (as bits)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Query blocks are issued last-first: under a causal mask the late rows hold the most live blocks,
  // and starting the longest rows first keeps the final wave short.
  // With q_ranges, (batch, head) bh computes only its query blocks [begin, begin + count): the unit of the
  // multi-GPU row sharding. The grid is sized for the largest count; the other CTAs leave at once.
  const int bh = blockIdx.y, h = bh % H;
  const int q_begin = q_ranges ? q_ranges[2 * bh] : 0;
  const int q_count = q_ranges ? min(q_ranges[2 * bh + 1], nq - q_begin) : (int)gridDim.x;
  if ((int)blockIdx.x >= q_count) return;
  const int qi = q_begin + q_count - 1 - (int)blockIdx.x;
  const size_t row_id = (size_t)bh * nq + qi;
  int cnt = valid[row_id];
  cnt = min(cnt, nk);

  if (cnt <= 0) {   // no live block: defined output (zeros)
    const int rows = min(128, N - qi * 128);
    constexpr int kChunks = D * (int)sizeof(OutT) / 16;
    OutT* obase = o + (size_t)(bh / H) * osb + (size_t)(bh % H) * osh + (size_t)qi * 128 * osn;
    for (int i = tid; i < rows * kChunks; i += kAttnThreads)
      reinterpret_cast<uint4*>(obase + (size_t)(i / kChunks) * osn)[i % kChunks] = make_uint4(0, 0, 0, 0);
    if (pv_count && tid < 4) pv_count[row_id * 4 + tid] = 0;
    return;
  }
  const int nsteps = (cnt + 1) >> 1;

  if (warp == 9) {
    tmem_alloc(&s_tmem_base, Shape::kTmemCols);
    tmem_relinquish();
  }
  if (tid == 256) {
    mbar_init(&bar_q, 1);
#pragma unroll
    for (int s = 0; s < SK; s++) {
      mbar_init(&bar_k_full[s], 1);
      mbar_init(&bar_k_empty[s], 1);
    }
#pragma unroll
    for (int s = 0; s < SV; s++) {
      mbar_init(&bar_v_full[s], 1);
      mbar_init(&bar_v_empty[s], 1);
    }
    mbar_init(&bar_s_full, 1);
    mbar_init(&bar_s_free, 8);     // one arrival per softmax warp
    mbar_init(&bar_p_ready, 8);
    mbar_init(&bar_o_done, 1);
    mbar_init(&bar_delta[0], 8);
    mbar_init(&bar_delta[1], 8);
    mbar_fence_init();
    s_skip[0] = 0;
    s_skip[1] = 0;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = s_tmem_base;
  const uint32_t tO = tbase + 128;
  const int32_t* lrow = lut + row_id * nk;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      mbar_arrive_expect_tx(&bar_q, Shape::kTileQ);
      tma_load_3d(sQ, &tmap_q, &bar_q, 0, qi * 128, bh);
    }
    // absolute block index of live entry n (n must not decrease between calls): prefix sums of the delta LUT,
    // 32 entries at a time, so that no load depends on the previous one
    const float* ksc = k_scale + (size_t)bh * nk;
    int win = -32, jabs = 0, jcarry = 0;
    float ks_lane = 0.f, ks_out = 0.f;      // K scale of this lane's entry / of the entry last returned
    auto block_of = [&](int n) -> int {
      if (n >= win + 32) {
        win = n & ~31;
        int incl = (win + lane < cnt) ? lrow[win + lane] : 0;
#pragma unroll
        for (int ofs = 1; ofs < 32; ofs <<= 1) {
          const int t = __shfl_up_sync(0xffffffffu, incl, ofs);
          if (lane >= ofs) incl += t;
        }
        jabs = jcarry + incl;
        jcarry = __shfl_sync(0xffffffffu, jabs, 31);
        jabs = max(0, min(jabs, nk - 1));
        ks_lane = ksc[jabs];
      }
      ks_out = __shfl_sync(0xffffffffu, ks_lane, n - win);
      return __shfl_sync(0xffffffffu, jabs, n - win);
    };
    int ok = 1, issued_k = 0, issued_v = 0, issued_tiles = 0;   // issued_tiles: K tiles requested in tile-ring mode
    auto load_pair = [&](const CUtensorMap* map, uint8_t* ring, uint64_t* full, uint64_t* empty, int stages, int s, int ja,
                         int jb, const int4* meta) {   // lane 0 only
      if (KT && meta) {   // K ring of single tiles: block n of the row's live list goes to slot n % 3
#pragma unroll
        for (int blk = 0; blk < 2; blk++) {
          if (blk == 1 && jb < 0) break;
          const int n = 2 * s + blk, ts = n % 3;
          if (n >= 3) ok = mbar_wait(&empty[ts], ((n / 3) - 1) & 1) ? 1 : 0;
          if (!ok) return;
          if (blk == 0) s_meta[s & 7] = *meta;   // see below: before the step's first K tile is requested
          mbar_arrive_expect_tx(&full[ts], Shape::kTileKV);
          tma_load_3d(ring + ts * Shape::kTileKV, map, &full[ts], 0, (blk ? jb : ja) * 64, bh);
          issued_tiles = n + 1;
        }
        return;
      }
      const int slot = s % stages;
      if (s >= stages) ok = mbar_wait(&empty[slot], ((s / stages) - 1) & 1) ? 1 : 0;
      if (!ok) return;
      // The step's block indices and K scales are published before its K tiles are requested: the softmax
      // warps read them once S of that step is complete, which is ordered after the tiles' arrival. The ring
      // slot was last used eight steps ago; the wait above has just shown that step s - stages has retired.
      if (meta) s_meta[s & 7] = *meta;
      if (PVF16 && !meta) {   // fp16 V: D/64 sub-tiles of 64 channels (128 bytes) per block
        uint8_t* dst = ring + slot * Shape::kPairV;
        mbar_arrive_expect_tx(&full[slot], (jb >= 0 ? 2 : 1) * Shape::kTileV);
#pragma unroll
        for (int nh = 0; nh < D / 64; nh++) {
          tma_load_3d(dst + nh * 8192, map, &full[slot], nh * 128, ja * 64, bh);
          if (jb >= 0) tma_load_3d(dst + Shape::kTileV + nh * 8192, map, &full[slot], nh * 128, jb * 64, bh);
        }
        return;
      }
      uint8_t* dst = ring + slot * Shape::kPairKV;
      mbar_arrive_expect_tx(&full[slot], (jb >= 0 ? 2 : 1) * Shape::kTileKV);
      tma_load_3d(dst, map, &full[slot], 0, ja * 64, bh);
      if (jb >= 0) tma_load_3d(dst + Shape::kTileKV, map, &full[slot], 0, jb * 64, bh);
    };
    int ja = block_of(0);
    float ka = ks_out, kb = 0.f;
    int jb = -1;
    if (cnt > 1) {
      jb = block_of(1);
      kb = ks_out;
    }
    if (lane == 0) {
      const int4 mt = make_int4(ja, max(jb, 0), __float_as_int(ka), __float_as_int(kb));
      load_pair(&tmap_k, sK, bar_k_full, bar_k_empty, SK, 0, ja, jb, &mt);
      issued_k = 1;
    }
    for (int s = 0; s < nsteps && ok; s++) {
      int na = -1, nb = -1;
      if (s + 1 < nsteps) {
        na = block_of(2 * s + 2);
        ka = ks_out;
        kb = 0.f;
        if (2 * s + 3 < cnt) {
          nb = block_of(2 * s + 3);
          kb = ks_out;
        }
      }
      if (lane == 0) {
        if (s + 1 < nsteps) {
          const int4 mt = make_int4(na, max(nb, 0), __float_as_int(ka), __float_as_int(kb));
          load_pair(&tmap_k, sK, bar_k_full, bar_k_empty, SK, s + 1, na, nb, &mt);
          if (ok) issued_k = s + 2;
        }
        if (ok) {
          load_pair(&tmap_v, sV, bar_v_full, bar_v_empty, SV, s, ja, jb, nullptr);
          if (ok) issued_v = s + 1;
        }
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      ja = na;
      jb = nb;
    }
    if (!ok && lane == 0) {
      report(dev_status, SPARGE_DEV_TIMEOUT_PRODUCER);
      // drain our own copies before the CTA's shared memory goes away
      if (KT) {
        for (int n = max(0, issued_tiles - 3); n < issued_tiles; n++) mbar_wait(&bar_k_full[n % 3], (n / 3) & 1);
      } else {
        for (int s = max(0, issued_k - SK); s < issued_k; s++) mbar_wait(&bar_k_full[s % SK], (s / SK) & 1);
      }
      for (int s = max(0, issued_v - SV); s < issued_v; s++) mbar_wait(&bar_v_full[s % SV], (s / SV) & 1);
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk2 = make_idesc(2, 1, 1, 0, 0, 128, 128);  // s32 += s8 * s8, both K-major, two blocks
      constexpr uint32_t idesc_qk1 = make_idesc(2, 1, 1, 0, 0, 128, 64);   // odd last block
      constexpr uint32_t idesc_pv = make_idesc(1, 0, 0, 0, 1, 128, D);     // f32 += e4m3 * e4m3, B MN-major
      constexpr uint32_t idesc_pv16 = make_idesc(1, 0, 0, 0, 1, 128, 64);  // f32 += f16 * f16, B MN-major, 64 channels
      constexpr uint32_t sbo = 8 * D;
      bool ok = mbar_wait(&bar_q, 0);
      // Every operand descriptor is built once: this thread shares its scheduler with four softmax warps,
      // and each instruction it spends between a hand-off and the MMAs it releases delays the other side.
      // A descriptor's low field is the address in 16-byte units, so moving to another ring slot is one add.
      uint64_t qd[D / 32], kd[D / 32], pd[4], vd[4];
#pragma unroll
      for (int ks = 0; ks < D / 32; ks++) {
        qd[ks] = make_smem_desc(smem_u32(sQ) + ks * 32, 16, sbo, Shape::kSwizzle);
        kd[ks] = make_smem_desc(smem_u32(sK) + ks * 32, 16, sbo, Shape::kSwizzle);
      }
#pragma unroll
      for (int ks = 0; ks < 4; ks++) {
        pd[ks] = make_smem_desc(smem_u32(sP) + ks * 32, 16, 1024, kSwizzle128B);
        vd[ks] = make_smem_desc(smem_u32(sV) + ks * 32 * D, 64 * D, sbo, Shape::kSwizzle);
      }
      constexpr uint64_t kSlotStep = (uint64_t)(Shape::kPairKV >> 4);
      // fp16 P.V of one block: per 64-channel sub-tile of V four instructions of 16 keys each
      auto issue_pv16 = [&](int blk, uint32_t slot_ofs_bytes, uint32_t& started) {
        const uint32_t pbase = smem_u32(sP) + blk * 16384, vbase = smem_u32(sV) + slot_ofs_bytes + blk * Shape::kTileV;
#pragma unroll
        for (int nh = 0; nh < D / 64; nh++) {
#pragma unroll
          for (int ks = 0; ks < 4; ks++)
            mma_f16_ss(tO + nh * 64, make_smem_desc(pbase + ks * 32, 16, 1024, kSwizzle128B),
                       make_smem_desc(vbase + nh * 8192 + ks * 2048, 8192, 1024, kSwizzle128B), idesc_pv16,
                       (ks > 0) ? 1u : started);
        }
        started = 1;
      };
      // waits for the K tiles of step s (one pair slot, or one or two tile slots of the tile ring)
      auto wait_k = [&](int s) -> bool {
        if (KT) {
          const int nblk = min(2, cnt - 2 * s);
          for (int blk = 0; blk < nblk; blk++) {
            const int n = 2 * s + blk;
            if (!mbar_wait(&bar_k_full[n % 3], (n / 3) & 1)) return false;
          }
          return true;
        }
        return mbar_wait(&bar_k_full[s % SK], (s / SK) & 1);
      };
      auto issue_qk = [&](int s) {   // the caller has waited for the K tiles of step s
        if (KT) {   // the step's tiles are not adjacent in the ring: one N = 64 instruction group per block
          tc_fence_after();
          const int nblk = min(2, cnt - 2 * s);
          for (int blk = 0; blk < nblk; blk++) {
            const int ts = (2 * s + blk) % 3;
            const uint64_t kofs = (uint64_t)ts * (uint64_t)(Shape::kTileKV >> 4);
#pragma unroll
            for (int ks = 0; ks < D / 32; ks++)
              mma_i8_ss(tbase + blk * 64, qd[ks], kd[ks] + kofs, idesc_qk1, ks > 0 ? 1u : 0u);
            tc_commit(&bar_k_empty[ts]);
          }
          tc_commit(&bar_s_full);
          return;
        }
        const int slot = s % SK;
        tc_fence_after();
        const uint64_t kofs = (uint64_t)slot * kSlotStep;
        const uint32_t idesc = (cnt - 2 * s >= 2) ? idesc_qk2 : idesc_qk1;
#pragma unroll
        for (int ks = 0; ks < D / 32; ks++) mma_i8_ss(tbase, qd[ks], kd[ks] + kofs, idesc, ks > 0 ? 1u : 0u);
        tc_commit(&bar_k_empty[slot]);
        tc_commit(&bar_s_full);
      };
      if (ok) ok = wait_k(0);
      if (ok) issue_qk(0);
      uint32_t o_started = 0;
      for (int s = 0; s < nsteps && ok; s++) {
        // Tiles arrive long before the softmax warps' hand-offs: their barriers are checked first, so that
        // only one wait stands between a hand-off and the MMAs it releases.
        if (s + 1 < nsteps) {
          ok = wait_k(s + 1);
          if (!ok) break;
          ok = mbar_wait(&bar_s_free, s & 1);      // every softmax warp has read S(s) into registers
          if (!ok) break;
          issue_qk(s + 1);
        }
        const int slot = s % SV;
        ok = mbar_wait(&bar_v_full[slot], (s / SV) & 1);
        if (!ok) break;
        const uint64_t vofs = (uint64_t)slot * kSlotStep;
        const int nb = min(2, cnt - 2 * s);
        ok = mbar_wait(&bar_p_ready, s & 1);
        if (!ok) break;
        tc_fence_after();
        if (PVF16) {
          if (!(PV_SKIP && s_skip[0])) issue_pv16(0, slot * Shape::kPairV, o_started);
          if (nb == 2 && !(PV_SKIP && s_skip[1])) issue_pv16(1, slot * Shape::kPairV, o_started);
        } else if (!(PV_SKIP && s_skip[0])) {
          mma_f8_ss(tO, pd[0], vd[0] + vofs, idesc_pv, o_started);
          mma_f8_ss(tO, pd[1], vd[1] + vofs, idesc_pv, 1u);
          o_started = 1;
        }
        if (!PVF16 && nb == 2 && !(PV_SKIP && s_skip[1])) {
          mma_f8_ss(tO, pd[2], vd[2] + vofs, idesc_pv, o_started);
          mma_f8_ss(tO, pd[3], vd[3] + vofs, idesc_pv, 1u);
          o_started = 1;
        }
        tc_commit(&bar_v_empty[slot]);
        tc_commit(&bar_o_done);
      }
      if (!ok) report(dev_status, SPARGE_DEV_TIMEOUT_MMA);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    // Two threads per query row (warps w and w + 4 share TMEM lanes 32 * (w & 3) ...): in a two-block step
    // thread `half` = 0 takes block A (S columns 0..63) and thread 1 block B (64..127); in an odd last step
    // they split the single block's 64 columns. Each thread works on its columns 32 at a time.
    const int half = warp >> 2, wq = warp & 3;
    const int row = wq * 32 + lane;
    const uint32_t tlane = (uint32_t)(wq * 32) << 16;
    const uint32_t tS = tbase + tlane;
    const int qrow = qi * 128 + row;
    const float qs = (GRAN3 ? q_scale[row_id * 32 + wq * 8 + (lane & 7)]
                            : q_scale[GRAN == 1 ? row_id : row_id * 4 + wq]) * sm_scale_log2;
    const float* ks_row = k_scale + (size_t)bh * nk * 4;   // GRAN3 only: four K scales per block
    const float thr = PV_SKIP ? pvthr[h] : 0.f;
    const uint32_t prow = smem_u32(sP) + (uint32_t)row * 128u;
    const int rsw = row & 7;
    float m = kMaskValue, d = 0.f;
    bool ok = true;
    int npv = 0;   // PV products issued for this query block (all of them unless the skip test fires)
    for (int s = 0; s < nsteps; s++) {
      const int nb = min(2, cnt - 2 * s);
      const int col0 = (nb == 2) ? half * 64 : half * 32;      // first S column of this thread
      const int nch = nb;                                       // 32-column chunks this thread handles
      ok = __all_sync(0xffffffffu, mbar_wait(&bar_s_full, s & 1));
      if (!ok) break;
      tc_fence_after();
      // this thread's block and scale (published by the producer warp before the step's K tiles were requested)
      const int4 mt = s_meta[s & 7];
      const bool second = (nb == 2) && half;
      const int j = second ? mt.y : mt.x;
      const float c = qs * __int_as_float(second ? mt.w : mt.z);
      float c4[4];
      if (GRAN3) {
        const float4 k4 = *reinterpret_cast<const float4*>(ks_row + (size_t)j * 4);
        c4[0] = qs * k4.x; c4[1] = qs * k4.y; c4[2] = qs * k4.z; c4[3] = qs * k4.w;
      }
      // per-key mask limit of this row inside the block: keys with block-local index >= klim are masked
      const int key0 = j * 64;
      const bool masked = (key0 + 64 > N) || (CAUSAL && (key0 + 63 > qi * 128));
      int klim = 64;
      if (masked) {
        klim = min(64, N - key0);
        if (CAUSAL) klim = min(klim, qrow - key0 + 1);
        klim = max(klim, 0);
      }
      const int kofs = col0 & 63;                                // block-local index of this thread's first column
      uint32_t sr[32];
      tmem_ld32(tS + col0, sr);
      tmem_wait_ld();
      float rmax = GRAN3 ? chunk_rowmax_g(sr, c4, klim - kofs)
                         : masked ? chunk_rowmax<true>(sr, c, klim - kofs) : chunk_rowmax<false>(sr, c, 32);
      if (nch == 2) {
        tmem_ld32(tS + col0 + 32, sr);
        tmem_wait_ld();
        rmax = fmaxf(rmax, GRAN3 ? chunk_rowmax_g(sr, c4, klim - kofs - 32)
                                 : masked ? chunk_rowmax<true>(sr, c, klim - kofs - 32) : chunk_rowmax<false>(sr, c, 32));
      }
      // exchange the partial row maxima of the two threads of a row
      s_rmax[s & 1][half][row] = rmax;
      pair_sync(1 + wq);
      const float r0 = s_rmax[s & 1][0][row], r1 = s_rmax[s & 1][1][row];
      const float m1 = fmaxf(m, r0);                              // two-block step: maximum after block A
      const float m2 = fmaxf(m1, r1);
      // PV-skip test (qk_int_sv_f8_cuda_sm89.cuh:317-353), per 64-key block as in the reference: block A is
      // tested against the running maximum before it, block B against the maximum after A. The warps
      // publish their partial maxima now and read the result only after the exponentials, so the reduction
      // latency is hidden; the last two live blocks are never skipped.
      const bool candA = PV_SKIP && (2 * s < cnt - 2), candB = PV_SKIP && (nb == 2) && (2 * s + 1 < cnt - 2);
      bool own_skip = false;   // per-warp mode: this warp's 32 rows drop their block (known before the exponentials)
      if (PV_SKIP && (candA || candB)) {
        // half 0 publishes block A's delta, half 1 block B's (a single-block step cannot be a candidate)
        const float w = warp_max(half ? (r1 - m1) : (r0 - m));
        if (lane == 0) {
          s_delta[s & 1][half][wq] = w;
          mbar_arrive(&bar_delta[s & 1]);
        }
        own_skip = pv_per_warp && (half ? candB : candA) && (w + thr <= 0.f);
      }
      const float alpha = (s > 0) ? ex2_approx(m - m2) : 0.f;
      const bool need_rescale = (s > 0) && __any_sync(0xffffffffu, m2 > m);
      // PV(s-1) must have retired before P is overwritten and before O is rescaled. (A second P buffer, which
      // takes this wait off all steps that do not rescale, was measured slower: the kernel is bound by issue
      // slots and the exponential unit together, not by this hand-off.)
      if (s > 0) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bar_o_done, (s - 1) & 1));
        if (!ok) break;
        if (need_rescale) {   // some row of this warp raised its maximum: this thread rescales its half of O
          tc_fence_after();
#pragma unroll
          for (int c0 = 0; c0 < D / 2; c0 += 16) {   // 16 columns at a time: 32 scores are still held in registers
            uint32_t ov[16];
            tmem_ld16(tO + tlane + half * (D / 2) + c0, ov);
            tmem_wait_ld();
            const float2 al2 = make_float2(alpha, alpha);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
              const float2 r2 = __fmul2_rn(make_float2(__uint_as_float(ov[i]), __uint_as_float(ov[i + 1])), al2);
              ov[i] = __float_as_uint(r2.x);
              ov[i + 1] = __float_as_uint(r2.y);
            }
            tmem_st16(tO + tlane + half * (D / 2) + c0, ov);
          }
          tmem_wait_st();
        }
      }
      d *= alpha;
      m = m2;
      // A 32-row group that drops its block in per-warp mode still writes its rows of P (as zeros, through the
      // masked path with no visible key): the other groups' rows of the same block may be multiplied.
      if (PV_SKIP && own_skip) klim = 0;
      const bool exact = masked || own_skip || !(c < kFastScaleLimit);
      // fp16 variant: this thread's block is sub-tile 0 or 1 of P, 8 keys per 16-byte chunk
      const uint32_t prow16 = smem_u32(sP) + (second ? 16384u : 0u) + (uint32_t)row * 128u;
      float sum = 0.f;
      if (nch == 2) {   // the second 32 columns are still in registers
        sum = PVF16 ? (exact ? chunk_exp_f16<true>(sr, c, m, klim - kofs - 32, one, prow16, (kofs >> 3) + 4, rsw)
                             : chunk_exp_f16<false>(sr, c, m, 32, one, prow16, (kofs >> 3) + 4, rsw))
              : GRAN3 ? chunk_exp_g(sr, c4, m, klim - kofs - 32, prow, (col0 >> 4) + 2, rsw)
              : exact ? chunk_exp<true>(sr, c, m, klim - kofs - 32, one, prow, (col0 >> 4) + 2, rsw)
                      : chunk_exp<false>(sr, c, m, 32, one, prow, (col0 >> 4) + 2, rsw);
        tmem_ld32(tS + col0, sr);            // the first 32 again: they did not stay in registers
        tmem_wait_ld();
      }
      // S has been read for the last time: the MMA warp may overwrite it with the next step's scores
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_s_free);
      sum += PVF16 ? (exact ? chunk_exp_f16<true>(sr, c, m, klim - kofs, one, prow16, kofs >> 3, rsw)
                            : chunk_exp_f16<false>(sr, c, m, 32, one, prow16, kofs >> 3, rsw))
             : GRAN3 ? chunk_exp_g(sr, c4, m, klim - kofs, prow, col0 >> 4, rsw)
             : exact ? chunk_exp<true>(sr, c, m, klim - kofs, one, prow, col0 >> 4, rsw)
                     : chunk_exp<false>(sr, c, m, 32, one, prow, col0 >> 4, rsw);
      bool skip = false;
      if (PV_SKIP && (candA || candB)) {
        ok = __all_sync(0xffffffffu, mbar_wait(&bar_delta[s & 1], (s >> 1) & 1));
        if (!ok) break;
        const float* da = s_delta[s & 1][0];
        const float* db = s_delta[s & 1][1];
        const bool skipA = candA && (fmaxf(fmaxf(da[0], da[1]), fmaxf(da[2], da[3])) + thr <= 0.f);
        const bool skipB = candB && (fmaxf(fmaxf(db[0], db[1]), fmaxf(db[2], db[3])) + thr <= 0.f);
        // candidates only occur in two-block steps: one block per thread. The product itself is left out only
        // when all four groups drop the block, which is the per-block decision in either mode.
        skip = pv_per_warp ? own_skip : (half ? skipB : skipA);
        if (tid == 0) {
          s_skip[0] = skipA ? 1 : 0;
          s_skip[1] = skipB ? 1 : 0;
        }
        // per-warp mode counts this warp's own block; the two warps of a group are added up at the end
        npv += pv_per_warp ? (own_skip ? 0 : 1) : (skipA ? 0 : 1) + (skipB ? 0 : 1);
      } else {
        if (PV_SKIP && tid == 0) {
          s_skip[0] = 0;
          s_skip[1] = 0;
        }
        npv += pv_per_warp ? (nb == 2 ? 1 : 1 - half) : nb;
      }
      if (!skip) d += sum;
      fence_proxy_async_smem();      // P bytes visible to the tensor core's operand fetch
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_p_ready);
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bar_o_done, (nsteps - 1) & 1));
    if (ok) {
      tc_fence_after();
      // total row sum = the two threads' partial sums
      s_rmax[0][half][row] = d;
      if (PV_SKIP && pv_per_warp) s_rmax[1][half][row] = __int_as_float(npv);
      pair_sync(1 + wq);
      // One count per 32-row group, the layout of the reference's PV_Count (qk_int_sv_f8_cuda_sm89.cuh:650-656).
      // With the per-block decision the four entries of a block are equal; with the per-warp decision each group
      // has its own, the sum of what its two warps (one per block of a pair) kept.
      if (PV_SKIP && pv_per_warp) npv = __float_as_int(s_rmax[1][0][row]) + __float_as_int(s_rmax[1][1][row]);
      if (pv_count && lane == 0 && half == 0) pv_count[row_id * 4 + wq] = npv;
      // A row that saw no key at all (token-level causal mask over every live block of its row of blocks) has an
      // empty sum: it is written as zeros. (The reference gives such a row the plain average of V over the masked
      // keys, because its mask value is a large finite number and exp2(mask - mask) = 1.)
      const float dsum = s_rmax[0][0][row] + s_rmax[0][1][row];
      const float inv = dsum > 0.f ? rcp_approx(dsum) : 0.f;
      const float* vs = PVF16 ? nullptr : v_scale + (size_t)bh * D + half * (D / 2);   // fp16 V carries no scale
      OutT* orow = o + (size_t)(bh / H) * osb + (size_t)(bh % H) * osh + (size_t)qrow * osn + half * (D / 2);
#pragma unroll
      for (int c0 = 0; c0 < D / 2; c0 += 32) {
        uint32_t ov[32];
        tmem_ld32(tO + tlane + half * (D / 2) + c0, ov);
        tmem_wait_ld();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
          const float a = __uint_as_float(ov[2 * i]) * inv * (PVF16 ? 1.f : vs[c0 + 2 * i]);
          const float bb = __uint_as_float(ov[2 * i + 1]) * inv * (PVF16 ? 1.f : vs[c0 + 2 * i + 1]);
          w[i] = pack2<OutT>(a, bb);
        }
        if (qrow < N) {
          uint4* dst = reinterpret_cast<uint4*>(orow + c0);
#pragma unroll
          for (int i = 0; i < 4; i++) dst[i] = make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]);
        }
      }
    } else if (lane == 0) {
      report(dev_status, SPARGE_DEV_TIMEOUT_SOFTMAX);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) tmem_dealloc(tbase, Shape::kTmemCols);
}

// ---------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = []() -> EncodeTiledFn {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return nullptr;
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// Byte tensor [planes, rows, inner] with a [1, box_rows, inner] box, swizzle span = inner bytes.
// box_inner: bytes of a row that one copy takes (default: the whole row); x coordinates are multiples of it.
static bool make_map(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t rows, uint64_t planes, uint32_t box_rows,
                     uint32_t box_inner = 0) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  if (box_inner == 0) box_inner = (uint32_t)inner;
  cuuint64_t dims[3] = {inner, rows, planes};
  cuuint64_t strides[2] = {inner, inner * rows};
  cuuint32_t box[3] = {box_inner, box_rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = box_inner == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, bool CAUSAL, int PV_MODE, typename OutT, int GRAN, bool PVF16 = false>
static int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, void* o, const int32_t* lut,
                       const int32_t* valid, const float* pvthr, const float* qs, const float* ks, const float* vs,
                       int32_t* status, int BH, int H, int N, float sm_scale_log2, long long osb, long long osh,
                       long long osn, int32_t* pv_count, const int32_t* q_ranges, int q_blocks_max, cudaStream_t st) {
  auto kern = attn_kernel<D, CAUSAL, PV_MODE, OutT, GRAN, PVF16>;
  constexpr int smem = AttnShape<D, PVF16>::kSmemBytes;
  // function attributes are per device: set on every call (cheap) rather than caching
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return SPARGE_ERR_CUDA;
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  const int nq = (N + 127) / 128, nk = (N + 63) / 64;
  const int gx = q_ranges ? min(q_blocks_max, nq) : nq;
  kern<<<dim3(gx, BH), kAttnThreads, smem, st>>>(tq, tk, tv, (OutT*)o, lut, valid, pvthr, qs, ks, vs, status, N, H, nq, nk,
                                                 sm_scale_log2, 1, osb, osh, osn, pv_count, q_ranges);
  return launch_status();
}

// One warp waits on an mbarrier that nobody arrives at, with a caller-chosen short limit, and reports
// the expiry through the same status word and code path as the attention kernel's bounded waits.
__global__ void wait_expiry_selftest_kernel(int32_t* dev_status, uint32_t slice_ns, uint32_t slices) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncthreads();
  const bool ok = mbar_wait(&bar, 0, slice_ns, slices);
  if (!ok && threadIdx.x == 0) report(dev_status, SPARGE_DEV_TIMEOUT_SOFTMAX);
}

}  // namespace sparge

extern "C" int sparge_selftest_wait_expiry(int32_t* dev_status, unsigned int slice_ns, unsigned int slices,
                                           sparge_stream_t stream) {
  if (!dev_status) return SPARGE_ERR_NULL;
  // a try lasts about 4 us even with a smaller hint: the test may not wait longer than 0.1 s either way
  if (slice_ns == 0 || slices == 0 || (unsigned long long)std::max(slice_ns, 4000u) * slices > 100000000ull)
    return SPARGE_ERR_INVALID_ARG;
  sparge::wait_expiry_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(dev_status, slice_ns, slices);
  return sparge::launch_status();
}

extern "C" int sparge_attn_fwd_gran(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o,
                                    const int32_t* lut, const int32_t* valid, const float* pvthreshd,
                                    const float* q_scale, const float* k_scale, const float* v_scale,
                                    int32_t* dev_status, int B, int H, int N, int D, int out_dtype, int is_causal,
                                    float sm_scale, long long o_stride_b, long long o_stride_h, long long o_stride_n,
                                    int32_t* pv_count, const int32_t* q_block_ranges, int q_blocks_max,
                                    int qk_quant_gran, int pv_threshold_mode, sparge_stream_t stream) {
  using namespace sparge;
  if (q_block_ranges && q_blocks_max <= 0) return SPARGE_ERR_INVALID_ARG;
  if (qk_quant_gran < 1 || qk_quant_gran > 3 || pv_threshold_mode < 0 || pv_threshold_mode > 2) return SPARGE_ERR_INVALID_ARG;
  if (pv_threshold_mode == 0) pvthreshd = nullptr;
  else if (!pvthreshd) return SPARGE_ERR_NULL;
  // per-thread K scales are read four at a time
  if (qk_quant_gran == 3 && (reinterpret_cast<uintptr_t>(k_scale) & 15)) return SPARGE_ERR_INVALID_ARG;

  if (!q_int8 || !k_int8 || !v8 || !o || !lut || !valid || !q_scale || !k_scale || !v_scale) return SPARGE_ERR_NULL;
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128) || (out_dtype != SPARGE_F16 && out_dtype != SPARGE_BF16))
    return SPARGE_ERR_INVALID_ARG;
  if (!(sm_scale > 0.f)) return SPARGE_ERR_INVALID_ARG;
  if ((long long)B * H > 65535) return SPARGE_ERR_TOO_LARGE;
  if (!strides_ok(o, o_stride_b, o_stride_h, o_stride_n)) return SPARGE_ERR_INVALID_ARG;
  const int BH = B * H;
  const int N_pad = (N + 127) / 128 * 128;
  CUtensorMap tq, tk, tv;
  if (!make_map(&tq, q_int8, D, N, BH, 128) || !make_map(&tk, k_int8, D, N, BH, 64) || !make_map(&tv, v8, D, N_pad, BH, 64))
    return SPARGE_ERR_CUDA;
  cudaStream_t st = (cudaStream_t)stream;
  const float sl2 = sm_scale * kLog2e;
  const bool causal = is_causal != 0, bf = out_dtype == SPARGE_BF16;
#define SPARGE_ATTN_G(DD, C, S, T, G) \
  launch_attn<DD, C, S, T, G>(tq, tk, tv, o, lut, valid, pvthreshd, q_scale, k_scale, v_scale, dev_status, BH, H, N, sl2, o_stride_b, o_stride_h, o_stride_n, pv_count, q_block_ranges, q_blocks_max, st)
#define SPARGE_ATTN(DD, C, S, T) \
  (qk_quant_gran == 3 ? SPARGE_ATTN_G(DD, C, S, T, 3) : qk_quant_gran == 2 ? SPARGE_ATTN_G(DD, C, S, T, 2) : SPARGE_ATTN_G(DD, C, S, T, 1))
#define SPARGE_ATTN_T(DD, C, S) (bf ? SPARGE_ATTN(DD, C, S, __nv_bfloat16) : SPARGE_ATTN(DD, C, S, __half))
#define SPARGE_ATTN_S(DD, C) \
  (pv_threshold_mode == 2 ? SPARGE_ATTN_T(DD, C, 2) : pv_threshold_mode == 1 ? SPARGE_ATTN_T(DD, C, 1) : SPARGE_ATTN_T(DD, C, 0))
#define SPARGE_ATTN_C(DD) (causal ? SPARGE_ATTN_S(DD, true) : SPARGE_ATTN_S(DD, false))
  return D == 64 ? SPARGE_ATTN_C(64) : SPARGE_ATTN_C(128);
#undef SPARGE_ATTN_C
#undef SPARGE_ATTN_S
#undef SPARGE_ATTN_T
#undef SPARGE_ATTN
#undef SPARGE_ATTN_G
}

extern "C" int sparge_attn_fwd_f16pv(const int8_t* q_int8, const int8_t* k_int8, const void* v_f16, void* o,
                                     const int32_t* lut, const int32_t* valid, const float* pvthreshd,
                                     const float* q_scale, const float* k_scale, int32_t* dev_status, int B, int H, int N,
                                     int D, int out_dtype, int is_causal, float sm_scale, long long o_stride_b,
                                     long long o_stride_h, long long o_stride_n, int32_t* pv_count,
                                     const int32_t* q_block_ranges, int q_blocks_max, sparge_stream_t stream) {
  using namespace sparge;
  if (q_block_ranges && q_blocks_max <= 0) return SPARGE_ERR_INVALID_ARG;
  if (!q_int8 || !k_int8 || !v_f16 || !o || !lut || !valid || !q_scale || !k_scale) return SPARGE_ERR_NULL;
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128) || (out_dtype != SPARGE_F16 && out_dtype != SPARGE_BF16))
    return SPARGE_ERR_INVALID_ARG;
  if (!(sm_scale > 0.f) || (reinterpret_cast<uintptr_t>(v_f16) & 15)) return SPARGE_ERR_INVALID_ARG;
  if ((long long)B * H > 65535) return SPARGE_ERR_TOO_LARGE;
  if (!strides_ok(o, o_stride_b, o_stride_h, o_stride_n)) return SPARGE_ERR_INVALID_ARG;
  const int BH = B * H;
  CUtensorMap tq, tk, tv;
  // V as bytes: rows of 2 D bytes, copied 128 bytes (64 channels) at a time; rows past N read as zeros
  if (!make_map(&tq, q_int8, D, N, BH, 128) || !make_map(&tk, k_int8, D, N, BH, 64) ||
      !make_map(&tv, v_f16, 2 * (uint64_t)D, N, BH, 64, 128))
    return SPARGE_ERR_CUDA;
  cudaStream_t st = (cudaStream_t)stream;
  const float sl2 = sm_scale * kLog2e;
  const bool causal = is_causal != 0, bf = out_dtype == SPARGE_BF16, skip = pvthreshd != nullptr;
#define SPARGE_F16PV(DD, C, S, T) \
  launch_attn<DD, C, S, T, 1, true>(tq, tk, tv, o, lut, valid, pvthreshd, q_scale, k_scale, nullptr, dev_status, BH, H, N, sl2, o_stride_b, o_stride_h, o_stride_n, pv_count, q_block_ranges, q_blocks_max, st)
#define SPARGE_F16PV_T(DD, C, S) (bf ? SPARGE_F16PV(DD, C, S, __nv_bfloat16) : SPARGE_F16PV(DD, C, S, __half))
#define SPARGE_F16PV_S(DD, C) (skip ? SPARGE_F16PV_T(DD, C, 1) : SPARGE_F16PV_T(DD, C, 0))
#define SPARGE_F16PV_C(DD) (causal ? SPARGE_F16PV_S(DD, true) : SPARGE_F16PV_S(DD, false))
  return D == 64 ? SPARGE_F16PV_C(64) : SPARGE_F16PV_C(128);
#undef SPARGE_F16PV_C
#undef SPARGE_F16PV_S
#undef SPARGE_F16PV_T
#undef SPARGE_F16PV
}

extern "C" int sparge_attn_fwd_rows(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o,
                                    const int32_t* lut, const int32_t* valid, const float* pvthreshd,
                                    const float* q_scale, const float* k_scale, const float* v_scale,
                                    int32_t* dev_status, int B, int H, int N, int D, int out_dtype, int is_causal,
                                    float sm_scale, long long o_stride_b, long long o_stride_h, long long o_stride_n,
                                    int32_t* pv_count, const int32_t* q_block_ranges, int q_blocks_max,
                                    sparge_stream_t stream) {
  return sparge_attn_fwd_gran(q_int8, k_int8, v8, o, lut, valid, pvthreshd, q_scale, k_scale, v_scale, dev_status, B, H, N, D,
                              out_dtype, is_causal, sm_scale, o_stride_b, o_stride_h, o_stride_n, pv_count, q_block_ranges,
                              q_blocks_max, 1, pvthreshd ? 1 : 0, stream);
}

extern "C" int sparge_attn_fwd_pv_count(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o,
                                        const int32_t* lut, const int32_t* valid, const float* pvthreshd,
                                        const float* q_scale, const float* k_scale, const float* v_scale,
                                        int32_t* dev_status, int B, int H, int N, int D, int out_dtype, int is_causal,
                                        float sm_scale, long long o_stride_b, long long o_stride_h, long long o_stride_n,
                                        int32_t* pv_count, sparge_stream_t stream) {
  return sparge_attn_fwd_rows(q_int8, k_int8, v8, o, lut, valid, pvthreshd, q_scale, k_scale, v_scale, dev_status, B, H, N, D,
                              out_dtype, is_causal, sm_scale, o_stride_b, o_stride_h, o_stride_n, pv_count, nullptr, 0, stream);
}

extern "C" int sparge_attn_fwd_strided(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o,
                                       const int32_t* lut, const int32_t* valid, const float* pvthreshd,
                                       const float* q_scale, const float* k_scale, const float* v_scale,
                                       int32_t* dev_status, int B, int H, int N, int D, int out_dtype, int is_causal,
                                       float sm_scale, long long o_stride_b, long long o_stride_h, long long o_stride_n,
                                       sparge_stream_t stream) {
  return sparge_attn_fwd_pv_count(q_int8, k_int8, v8, o, lut, valid, pvthreshd, q_scale, k_scale, v_scale, dev_status, B, H,
                                  N, D, out_dtype, is_causal, sm_scale, o_stride_b, o_stride_h, o_stride_n, nullptr, stream);
}

extern "C" int sparge_attn_fwd(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o,
                               const int32_t* lut, const int32_t* valid, const float* pvthreshd, const float* q_scale,
                               const float* k_scale, const float* v_scale, int32_t* dev_status, int B, int H, int N,
                               int D, int out_dtype, int is_causal, float sm_scale, sparge_stream_t stream) {
  return sparge_attn_fwd_strided(q_int8, k_int8, v8, o, lut, valid, pvthreshd, q_scale, k_scale, v_scale, dev_status, B, H,
                                 N, D, out_dtype, is_causal, sm_scale, (long long)H * N * D, (long long)N * D, D, stream);
}
