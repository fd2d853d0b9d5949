// LUT-driven block-sparse attention for sm_100a.
//   S = Q8 K8^T   : tcgen05.mma kind::i8, operands staged by TMA into 128B/64B-swizzled smem,
//                   s32 accumulator in tensor memory (TMEM)
//   online softmax in registers (one thread per query row, no shuffles), P rounded to e4m3 and
//                   written back into the TMEM columns S came from
//   O += P8 V8    : tcgen05.mma kind::f8f6f4 with A = P from TMEM, B = V tile (token-major,
//                   MN-major descriptor), f32 accumulator in TMEM
// Replaces qk_int_sv_f8_block_sparse_attn_kernel (csrc/qattn/qk_int_sv_f8_cuda_sm89.cuh:42-755)
// and its host wrapper (csrc/qattn/qk_int_sv_f8_cuda_sm89.cu:392-585).
//
// One CTA per (q-block of 128 rows, head, batch); 6 warps:
//   warps 0-3  softmax / correction / epilogue (thread t owns query row t = TMEM lane t)
//   warp  4    TMA producer: walks the delta-encoded LUT and fetches only live K/V blocks
//   warp  5    MMA issuer (one elected lane) and TMEM owner
// TMEM columns: [0,64) S0/P0, [64,128) S1/P1, [128,128+D) O  -> 256 columns, two CTAs per SM.
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


template <int D>
struct AttnShape {
  static constexpr int kStages = (D == 128) ? 5 : 8;
  static constexpr int kTileQ = 128 * D;
  static constexpr int kTileKV = 64 * D;
  static constexpr int kSmemBytes = 1024 + kTileQ + kStages * 2 * kTileKV;
  static constexpr int kTmemCols = 256;
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

template <int D, bool CAUSAL, bool PV_SKIP, typename OutT>
__global__ void __launch_bounds__(192, 2)
attn_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
            const __grid_constant__ CUtensorMap tmap_v, OutT* __restrict__ o, const int32_t* __restrict__ lut,
            const int32_t* __restrict__ valid, const float* __restrict__ pvthr, const float* __restrict__ q_scale,
            const float* __restrict__ k_scale, const float* __restrict__ v_scale, int32_t* dev_status, int N, int H,
            int nq, int nk, float sm_scale_log2, int one, long long osb, long long osh, long long osn,
            int32_t* __restrict__ pv_count) {
  using Shape = AttnShape<D>;
  constexpr int STAGES = Shape::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = smem + Shape::kTileQ;   // stage s: K at sKV + s*2*kTileKV, V right after it

  __shared__ uint64_t bar_q, bar_kv_full[STAGES], bar_kv_empty[STAGES], bar_s_full[2], bar_p_ready[2], bar_o_done,
      bar_delta[2];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_skip[2];
  __shared__ float s_delta[2][4];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // Query blocks are issued last-first: under a causal mask the late rows hold the most live blocks,
  // and starting the longest rows first keeps the final wave short.
  const int qi = (int)gridDim.x - 1 - (int)blockIdx.x, bh = blockIdx.y, h = bh % H;
  const size_t row_id = (size_t)bh * nq + qi;
  int cnt = valid[row_id];
  cnt = min(cnt, nk);

  if (cnt <= 0) {   // no live block: defined output (zeros)
    const int rows = min(128, N - qi * 128);
    constexpr int kChunks = D * (int)sizeof(OutT) / 16;
    OutT* obase = o + (size_t)(bh / H) * osb + (size_t)(bh % H) * osh + (size_t)qi * 128 * osn;
    for (int i = tid; i < rows * kChunks; i += 192)
      reinterpret_cast<uint4*>(obase + (size_t)(i / kChunks) * osn)[i % kChunks] = make_uint4(0, 0, 0, 0);
    if (pv_count && tid < 4) pv_count[row_id * 4 + tid] = 0;
    return;
  }

  if (warp == 5) {
    tmem_alloc(&s_tmem_base, Shape::kTmemCols);
    tmem_relinquish();
  }
  if (tid == 128) {
    mbar_init(&bar_q, 1);
#pragma unroll
    for (int s = 0; s < STAGES; s++) {
      mbar_init(&bar_kv_full[s], 1);
      mbar_init(&bar_kv_empty[s], 1);
    }
    mbar_init(&bar_s_full[0], 1);
    mbar_init(&bar_s_full[1], 1);
    mbar_init(&bar_p_ready[0], 4);    // one arrival per softmax warp
    mbar_init(&bar_p_ready[1], 4);
    mbar_init(&bar_o_done, 1);
    mbar_init(&bar_delta[0], 4);
    mbar_init(&bar_delta[1], 4);
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

  if (warp == 4) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      mbar_arrive_expect_tx(&bar_q, Shape::kTileQ);
      tma_load_3d(sQ, &tmap_q, &bar_q, 0, qi * 128, bh);
    }
    int jbase = 0, issued = 0;
    int ok = 1;
    for (int n0 = 0; n0 < cnt && ok; n0 += 32) {
      const int n = n0 + lane;
      int incl = (n < cnt) ? lrow[n] : 0;
#pragma unroll
      for (int ofs = 1; ofs < 32; ofs <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, incl, ofs);
        if (lane >= ofs) incl += t;
      }
      const int jabs = jbase + incl;
      jbase = __shfl_sync(0xffffffffu, jabs, 31);
      const int lim = min(32, cnt - n0);
      for (int kk = 0; kk < lim; kk++) {
        int j = __shfl_sync(0xffffffffu, jabs, kk);
        j = max(0, min(j, nk - 1));
        if (lane == 0) {
          const int nn = n0 + kk, s = nn % STAGES;
          if (nn >= STAGES) ok = mbar_wait(&bar_kv_empty[s], ((nn / STAGES) - 1) & 1) ? 1 : 0;
          if (ok) {
            uint8_t* dK = sKV + s * 2 * Shape::kTileKV;
            mbar_arrive_expect_tx(&bar_kv_full[s], 2 * Shape::kTileKV);
            tma_load_3d(dK, &tmap_k, &bar_kv_full[s], 0, j * 64, bh);
            tma_load_3d(dK + Shape::kTileKV, &tmap_v, &bar_kv_full[s], 0, j * 64, bh);
            issued = nn + 1;
          }
        }
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
      }
    }
    if (!ok && lane == 0) {
      report(dev_status, SPARGE_DEV_TIMEOUT_PRODUCER);
      // drain our own copies before the CTA's shared memory goes away
      for (int nn = max(0, issued - STAGES); nn < issued; nn++) mbar_wait(&bar_kv_full[nn % STAGES], (nn / STAGES) & 1);
    }
  } else if (warp == 5) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = make_idesc(2, 1, 1, 0, 0, 128, 64);   // s32 += s8 * s8, both K-major
      constexpr uint32_t idesc_pv = make_idesc(1, 0, 0, 0, 1, 128, D);    // f32 += e4m3 * e4m3, B MN-major
      constexpr uint32_t sbo = 8 * D;
      bool ok = mbar_wait(&bar_q, 0);
      auto issue_pv = [&](int m) {
        const int b = m & 1, s = m % STAGES;
        ok = mbar_wait(&bar_p_ready[b], (m >> 1) & 1);
        if (!ok) return;
        tc_fence_after();
        if (!(PV_SKIP && s_skip[b])) {
          const uint32_t vaddr = smem_u32(sKV + s * 2 * Shape::kTileKV + Shape::kTileKV);
#pragma unroll
          for (int ks = 0; ks < 2; ks++) {
            const uint64_t bd = make_smem_desc(vaddr + ks * 32 * D, 64 * D, sbo, Shape::kSwizzle);
            mma_f8_ts(tO, tbase + b * 64 + ks * 8, bd, idesc_pv, (m > 0 || ks > 0) ? 1u : 0u);
          }
        }
        tc_commit(&bar_kv_empty[s]);
        tc_commit(&bar_o_done);
      };
      for (int n = 0; n < cnt && ok; n++) {
        const int s = n % STAGES;
        ok = mbar_wait(&bar_kv_full[s], (n / STAGES) & 1);
        if (!ok) break;
        tc_fence_after();
        const uint32_t qaddr = smem_u32(sQ), kaddr = smem_u32(sKV + s * 2 * Shape::kTileKV);
#pragma unroll
        for (int ks = 0; ks < D / 32; ks++) {
          const uint64_t ad = make_smem_desc(qaddr + ks * 32, 16, sbo, Shape::kSwizzle);
          const uint64_t bd = make_smem_desc(kaddr + ks * 32, 16, sbo, Shape::kSwizzle);
          mma_i8_ss(tbase + (n & 1) * 64, ad, bd, idesc_qk, ks > 0 ? 1u : 0u);
        }
        tc_commit(&bar_s_full[n & 1]);
        if (n > 0) issue_pv(n - 1);
      }
      if (ok) issue_pv(cnt - 1);
      if (!ok) report(dev_status, SPARGE_DEV_TIMEOUT_MMA);
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax / correction / epilogue
    const uint32_t tlane = (uint32_t)(warp * 32) << 16;
    const int qrow = qi * 128 + tid;
    const float qs = q_scale[row_id] * sm_scale_log2;
    const float thr = PV_SKIP ? pvthr[h] : 0.f;
    const float* ksc = k_scale + (size_t)bh * nk;
    // `one` is a kernel argument equal to 1 that the compiler cannot fold: multiplying by it turns the
    // int->float bias add into an IMAD, which issues on the FMA pipe instead of the half-rate integer pipe.
    float m = kMaskValue, d = 0.f;
    // Software-pipelined metadata: the LUT delta is loaded two iterations ahead and the K scale one
    // iteration ahead, and neither value is touched before the iteration after its load, so the two
    // dependent global loads never stall the in-order issue of this warp.
    int j_cur = max(0, min(lrow[0], nk - 1));
    float ks_cur = ksc[j_cur];
    int j_nxt = max(0, min(j_cur + ((cnt > 1) ? lrow[1] : 0), nk - 1));
    float ks_nxt = ksc[j_nxt];
    int delta_nn = (cnt > 2) ? lrow[2] : 0;
    bool ok = true;
    int npv = 0;   // PV products issued for this query block (all of them unless the skip test fires)
    for (int n = 0; n < cnt; n++) {
      const int j = j_cur;
      const float c = qs * ks_cur;
      j_cur = j_nxt;
      ks_cur = ks_nxt;
      j_nxt = max(0, min(j_nxt + delta_nn, nk - 1));
      ks_nxt = ksc[j_nxt];                                 // consumed in iteration n+2
      delta_nn = (n + 3 < cnt) ? lrow[n + 3] : 0;          // consumed in iteration n+1
      const int b = n & 1;
      const uint32_t tS = tbase + b * 64 + tlane;
      ok = mbar_wait(&bar_s_full[b], (n >> 1) & 1);
      if (!ok) break;
      tc_fence_after();
      uint32_t sr[64];
      tmem_ld32(tS, sr);
      tmem_ld32(tS + 32, sr + 32);
      tmem_wait_ld();
      const int key0 = j * 64;
      const bool masked_block = (key0 + 64 > N) || (CAUSAL && (key0 + 63 > qi * 128));
      // per-key mask limit for this row: keys with local index >= klim are masked
      int klim = 64;
      if (masked_block) {
        klim = min(64, N - key0);
        if (CAUSAL) klim = min(klim, qrow - key0 + 1);
        klim = max(klim, 0);
      }
      float rmax;
      if (!masked_block) {
        int m0 = (int)sr[0], m1 = (int)sr[16], m2 = (int)sr[32], m3 = (int)sr[48];   // four chains: short latency
#pragma unroll
        for (int k = 1; k < 15; k += 2) {
          m0 = __vimax3_s32(m0, (int)sr[k], (int)sr[k + 1]);
          m1 = __vimax3_s32(m1, (int)sr[16 + k], (int)sr[16 + k + 1]);
          m2 = __vimax3_s32(m2, (int)sr[32 + k], (int)sr[32 + k + 1]);
          m3 = __vimax3_s32(m3, (int)sr[48 + k], (int)sr[48 + k + 1]);
        }
        m0 = __vimax3_s32(m0, m1, (int)sr[15]);
        m2 = __vimax3_s32(m2, m3, (int)sr[31]);
        const int mx = max(__vimax3_s32(m0, m2, (int)sr[47]), (int)sr[63]);
        rmax = (__int_as_float(mx + (int)kMagicBits) - kMagic) * c;   // c > 0: max commutes with the scaling
      } else {
        int mx = INT_MIN;
#pragma unroll
        for (int k = 0; k < 64; k++) mx = (k < klim) ? max(mx, (int)sr[k]) : mx;
        rmax = (klim > 0) ? __int2float_rn(mx) * c : kMaskValue;
      }
      const float m_new = fmaxf(m, rmax);
      // PV-skip test (qk_int_sv_f8_cuda_sm89.cuh:317-353): the block is skipped when, over all 128 rows,
      // max(row maximum - running maximum) + threshold <= 0. The four warps publish their partial maxima
      // now and read the result only after the exponentials, so the reduction latency is hidden; a block
      // that turns out to be skipped has wasted its exponentials (rare) but leaves no trace: its row sums
      // are dropped and the MMA warp does not issue its PV product.
      const bool skip_candidate = PV_SKIP && n < cnt - 2;   // the last two live blocks are never skipped
      if (skip_candidate) {
        const float wmax = warp_max(rmax - m);
        if (lane == 0) {
          s_delta[b][warp] = wmax;
          mbar_arrive(&bar_delta[b]);
        }
      }
      // Rescaling of the running output is deferred until after the exponentials: by then PV(n-1) has
      // normally retired, so the wait below does not stall. The wait itself is unconditional: a parity
      // wait only tells phases apart if every phase of the barrier is observed in order.
      const float alpha = (n > 0) ? ex2_approx(m - m_new) : 0.f;
      const bool need_rescale = (n > 0) && __any_sync(0xffffffffu, m_new > m);
      auto settle_output = [&]() -> bool {
        if (n > 0) {
          if (!mbar_wait(&bar_o_done, (n - 1) & 1)) return false;
          if (need_rescale) {   // some row of this warp raised its maximum
            tc_fence_after();
#pragma unroll
            for (int c0 = 0; c0 < D; c0 += 32) {
              uint32_t ov[32];
              tmem_ld32(tO + tlane + c0, ov);
              tmem_wait_ld();
              const float2 al2 = make_float2(alpha, alpha);
#pragma unroll
              for (int i = 0; i < 32; i += 2) {
                const float2 r2 = __fmul2_rn(make_float2(__uint_as_float(ov[i]), __uint_as_float(ov[i + 1])), al2);
                ov[i] = __float_as_uint(r2.x);
                ov[i + 1] = __float_as_uint(r2.y);
              }
              tmem_st32(tO + tlane + c0, ov);
            }
            tmem_wait_st();
          }
        }
        return true;
      };
      d *= alpha;
      m = m_new;
      uint32_t pr[16];
      float sum;
      if (!masked_block && c < kFastScaleLimit) {
        // int32 -> fp32 by adding the bit pattern of 1.5 * 2^23 (exact for |S| < 2^22; here |S| <= 127^2 * 128);
        // the 2^23 bias is taken out again inside the FMA constant. Packed f32x2 FMA / ADD halve the issue slots.
        // That constant is rounded at the magnitude of 1.5 * 2^23 * c, so the exponents of this block are off
        // by a common amount of at most 0.75 * c: blocks whose scale is not small take the exact path below.
        const float off = fmaf(-kMagic, c, kFp8Offset - m);
        const float2 c2 = make_float2(c, c), o2 = make_float2(off, off);
        float2 s0 = make_float2(0.f, 0.f), s1 = make_float2(0.f, 0.f);
#pragma unroll
        for (int k = 0; k < 64; k += 4) {
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
          pr[k >> 2] = cvt_e4m3x4(a.x, a.y, bb.x, bb.y);
          // P goes to TMEM four words at a time, as soon as they exist, instead of being parked in 16
          // registers until the end of the block.
          if ((k & 12) == 12) tmem_st4(tS + (k >> 2) - 3, pr + (k >> 2) - 3);
        }
        s0 = __fadd2_rn(s0, s1);
        sum = s0.x + s0.y;
      } else {
        const float off = kFp8Offset - m;
        sum = 0.f;
#pragma unroll
        for (int k = 0; k < 64; k += 4) {
          float p0 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 0]), c, off));
          float p1 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 1]), c, off));
          float p2 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 2]), c, off));
          float p3 = ex2_approx(fmaf(__int2float_rn((int)sr[k + 3]), c, off));
          p0 = (k + 0 < klim) ? p0 : 0.f;
          p1 = (k + 1 < klim) ? p1 : 0.f;
          p2 = (k + 2 < klim) ? p2 : 0.f;
          p3 = (k + 3 < klim) ? p3 : 0.f;
          sum += (p0 + p1) + (p2 + p3);
          pr[k >> 2] = cvt_e4m3x4(p0, p1, p2, p3);
        }
        tmem_st16(tS, pr);
      }
      bool skip = false;
      if (skip_candidate) {
        ok = mbar_wait(&bar_delta[b], (n >> 1) & 1);
        if (!ok) break;
        const float dcta = fmaxf(fmaxf(s_delta[b][0], s_delta[b][1]), fmaxf(s_delta[b][2], s_delta[b][3]));
        skip = (dcta + thr <= 0.f);
      }
      if (!skip) {
        d += sum;
        npv++;
      }
      ok = settle_output();
      if (!ok) break;
      tmem_wait_st();   // P of a skipped block is stored too; its PV product is simply never issued
      if (PV_SKIP && tid == 0) s_skip[b] = skip ? 1 : 0;
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&bar_p_ready[b]);
    }
    if (ok) ok = mbar_wait(&bar_o_done, (cnt - 1) & 1);
    if (ok) {
      tc_fence_after();
      // One count per 32-row group, the layout of the reference's PV_Count (qk_int_sv_f8_cuda_sm89.cuh:650-656);
      // the skip decision is taken per block, so the four entries of a block are equal.
      if (pv_count && lane == 0) pv_count[row_id * 4 + warp] = npv;
      const float inv = rcp_approx(d);
      const float* vs = v_scale + (size_t)bh * D;
      OutT* orow = o + (size_t)(bh / H) * osb + (size_t)(bh % H) * osh + (size_t)qrow * osn;
#pragma unroll
      for (int c0 = 0; c0 < D; c0 += 32) {
        uint32_t ov[32];
        tmem_ld32(tO + tlane + c0, ov);
        tmem_wait_ld();
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; i++) {
          const float a = __uint_as_float(ov[2 * i]) * inv * vs[c0 + 2 * i];
          const float bb = __uint_as_float(ov[2 * i + 1]) * inv * vs[c0 + 2 * i + 1];
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
  if (warp == 5) tmem_dealloc(tbase, Shape::kTmemCols);
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
static bool make_map(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t rows, uint64_t planes, uint32_t box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return false;
  cuuint64_t dims[3] = {inner, rows, planes};
  cuuint64_t strides[2] = {inner, inner * rows};
  cuuint32_t box[3] = {(cuuint32_t)inner, box_rows, 1};
  cuuint32_t es[3] = {1, 1, 1};
  const CUtensorMapSwizzle sw = inner == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  return enc(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(ptr), dims, strides, box, es,
             CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int D, bool CAUSAL, bool PV_SKIP, typename OutT>
static int launch_attn(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, void* o, const int32_t* lut,
                       const int32_t* valid, const float* pvthr, const float* qs, const float* ks, const float* vs,
                       int32_t* status, int BH, int H, int N, float sm_scale_log2, long long osb, long long osh,
                       long long osn, int32_t* pv_count, cudaStream_t st) {
  auto kern = attn_kernel<D, CAUSAL, PV_SKIP, OutT>;
  constexpr int smem = AttnShape<D>::kSmemBytes;
  // function attributes are per device: set on every call (cheap) rather than caching
  if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return SPARGE_ERR_CUDA;
  cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  const int nq = (N + 127) / 128, nk = (N + 63) / 64;
  kern<<<dim3(nq, BH), 192, smem, st>>>(tq, tk, tv, (OutT*)o, lut, valid, pvthr, qs, ks, vs, status, N, H, nq, nk,
                                        sm_scale_log2, 1, osb, osh, osn, pv_count);
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
  if (slice_ns == 0 || slices == 0 || (unsigned long long)slice_ns * slices > 100000000ull) return SPARGE_ERR_INVALID_ARG;
  sparge::wait_expiry_selftest_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(dev_status, slice_ns, slices);
  return sparge::launch_status();
}

extern "C" int sparge_attn_fwd_pv_count(const int8_t* q_int8, const int8_t* k_int8, const uint8_t* v8, void* o,
                                        const int32_t* lut, const int32_t* valid, const float* pvthreshd,
                                        const float* q_scale, const float* k_scale, const float* v_scale,
                                        int32_t* dev_status, int B, int H, int N, int D, int out_dtype, int is_causal,
                                        float sm_scale, long long o_stride_b, long long o_stride_h, long long o_stride_n,
                                        int32_t* pv_count, sparge_stream_t stream) {
  using namespace sparge;
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
  const bool causal = is_causal != 0, skip = pvthreshd != nullptr, bf = out_dtype == SPARGE_BF16;
#define SPARGE_ATTN(DD, C, S, T) \
  launch_attn<DD, C, S, T>(tq, tk, tv, o, lut, valid, pvthreshd, q_scale, k_scale, v_scale, dev_status, BH, H, N, sl2, o_stride_b, o_stride_h, o_stride_n, pv_count, st)
#define SPARGE_ATTN_T(DD, C, S) (bf ? SPARGE_ATTN(DD, C, S, __nv_bfloat16) : SPARGE_ATTN(DD, C, S, __half))
#define SPARGE_ATTN_S(DD, C) (skip ? SPARGE_ATTN_T(DD, C, true) : SPARGE_ATTN_T(DD, C, false))
#define SPARGE_ATTN_C(DD) (causal ? SPARGE_ATTN_S(DD, true) : SPARGE_ATTN_S(DD, false))
  return D == 64 ? SPARGE_ATTN_C(64) : SPARGE_ATTN_C(128);
#undef SPARGE_ATTN_C
#undef SPARGE_ATTN_S
#undef SPARGE_ATTN_T
#undef SPARGE_ATTN
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
