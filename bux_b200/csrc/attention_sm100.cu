// Softmax attention for sm_100a on tcgen05 tensor cores, forward pass.
//
// One CTA per (batch, query head, 128-query tile); 192 threads:
//   warps 0..3  softmax: one query row per thread. Reads S = Q·K^T from tensor memory
//               (tcgen05.ld), keeps the running max / sum, writes P (bf16) into shared
//               memory in the tensor core's swizzled K-major layout, and accumulates
//               P·V (read back from tensor memory) into fp32 registers.
//   warp 4      TMA producer: Q once, then K/V tiles into a 2-stage ring (plain TMA
//               loads, no multicast).
//   warp 5      MMA issuer: S_j = Q·K_j^T into one of two TMEM buffers, then
//               PV_j = P_j·V_j; S_{j+1} is issued before PV_j so the tensor core
//               works while the softmax warps run.
// GQA (H % G == 0), causal with bottom-right alignment, sliding window and attention
// sinks (one extra logit per head in the denominator) are handled in the mask / final
// normalisation. Fully masked key tiles are skipped.
//
// Reference counterparts: cuDNN SDPA and FlashAttention-4 behind parallel/flash.py:573-678
// and parallel/fa4.py:410-573; the math is that of parallel/context.py:130 (xla).
#include "attention_sm100.h"
#include "common.cuh"
#include "gemm_sm100.h"

namespace bux {

constexpr int KID_ATTN_FWD = 2;
constexpr int QT = 128;  // query rows per CTA
constexpr int KT = 128;  // keys per tile
constexpr int ATTN_THREADS = 192;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct AttnFwdParams {
  alignas(64) CUtensorMap tmap_q;
  alignas(64) CUtensorMap tmap_kv_k;
  alignas(64) CUtensorMap tmap_kv_v;
  void* o; float* lse; const float* sinks; Status* status;
  int B, T, S, H, G;
  float scale_log2; int causal, window;
};

template <int D>
struct AttnFwdCfg {
  static constexpr int DC = D / 64;               // 64-column chunks of the head dim
  static constexpr int TILE_BYTES = DC * 16384;   // one [128 x D] bf16 tile
  static constexpr int P_BYTES = 2 * 16384;       // [128 x 128] bf16
  static constexpr int SMEM_BYTES = TILE_BYTES * 5 + P_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;           // S0, S1 (128 each), PV (D)
};

template <int D>
__global__ void __launch_bounds__(ATTN_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ AttnFwdParams p) {
  using Cfg = AttnFwdCfg<D>;
  constexpr int DC = Cfg::DC;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::TILE_BYTES;              // 2 stages
  uint8_t* sV = sK + 2 * Cfg::TILE_BYTES;          // 2 stages
  uint8_t* sP = sV + 2 * Cfg::TILE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + Cfg::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;    // [2]
  uint64_t* kv_empty = bars + 3;   // [2]
  uint64_t* s_full = bars + 5;     // [2]
  uint64_t* p_ready = bars + 7;
  uint64_t* pv_full = bars + 8;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_qt = (p.T + QT - 1) / QT;
  const int qt = n_qt - 1 - blockIdx.x;  // long (late) rows first under a causal mask
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.H / p.G);
  const int q0 = qt * QT;
  const int shift = p.S - p.T;  // bottom-right alignment of the causal diagonal
  // key tiles this query tile can see
  int j_hi = (p.S + KT - 1) / KT;
  if (p.causal) j_hi = min(j_hi, (q0 + QT - 1 + shift) / KT + 1);
  int j_lo = 0;
  if (p.window > 0) j_lo = max(0, (q0 + shift - p.window + 1) / KT);
  const int n_tiles = max(0, j_hi - j_lo);
  Status* st = p.status;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); mbar_init(&s_full[i], 1); }
    mbar_init(p_ready, 128);
    mbar_init(pv_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 5) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s = tmem_base;        // two 128-column buffers
  const uint32_t tmem_pv = tmem_base + 256;

  if (warp == 4) {
    // -------------------------------------------------------------- TMA producer
    if (elect_one() && n_tiles > 0) {
      mbar_expect_tx(q_full, Cfg::TILE_BYTES);
      for (int c = 0; c < DC; ++c)
        tma_load_2d(sQ + c * 16384, &p.tmap_q, h * D + c * 64, b * p.T + q0, q_full);
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t & 1;
        if (!mbar_wait(&kv_empty[s], ((t >> 1) & 1) ^ 1, abort_flag, st, KID_ATTN_FWD, 1)) break;
        mbar_expect_tx(&kv_full[s], 2 * Cfg::TILE_BYTES);
        const int row = b * p.S + (j_lo + t) * KT;
        for (int c = 0; c < DC; ++c) {
          tma_load_2d(sK + s * Cfg::TILE_BYTES + c * 16384, &p.tmap_kv_k, g * D + c * 64, row, &kv_full[s]);
          tma_load_2d(sV + s * Cfg::TILE_BYTES + c * 16384, &p.tmap_kv_v, g * D + c * 64, row, &kv_full[s]);
        }
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one() && n_tiles > 0) {
      const uint32_t idesc_s = make_idesc(FMT_BF16, FMT_BF16, 128, KT, false, false);
      const uint32_t idesc_pv = make_idesc(FMT_BF16, FMT_BF16, 128, D, false, true);
      auto issue_s = [&](int t) {
        const int s = t & 1;
        const uint32_t a0 = smem_u32(sQ), b0 = smem_u32(sK + s * Cfg::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_f16(tmem_s + s * 128, make_smem_desc(a0 + off, 0, 1024, 2), make_smem_desc(b0 + off, 0, 1024, 2), idesc_s, kk > 0);
        }
        tc_commit(&s_full[s]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, st, KID_ATTN_FWD, 2);
      ok = ok && mbar_wait(&kv_full[0], 0, abort_flag, st, KID_ATTN_FWD, 3);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        for (int t = 0; t < n_tiles && ok; ++t) {
          if (t + 1 < n_tiles) {
            ok = mbar_wait(&kv_full[(t + 1) & 1], ((t + 1) >> 1) & 1, abort_flag, st, KID_ATTN_FWD, 4);
            if (!ok) break;
            tc_fence_after();
            issue_s(t + 1);
          }
          ok = mbar_wait(p_ready, t & 1, abort_flag, st, KID_ATTN_FWD, 5);
          if (!ok) break;
          tc_fence_after();
          const int s = t & 1;
          const uint32_t a0 = smem_u32(sP), b0 = smem_u32(sV + s * Cfg::TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < KT / 16; ++kk) {
            const uint64_t ad = make_smem_desc(a0 + (kk >> 2) * 16384 + (kk & 3) * 32, 0, 1024, 2);
            const uint64_t bd = make_smem_desc(b0 + kk * 2048, 16384, 1024, 2);
            mma_f16(tmem_pv, ad, bd, idesc_pv, kk > 0);
          }
          tc_commit(pv_full);
          tc_commit(&kv_empty[s]);
        }
      }
    }
  } else {
    // -------------------------------------------------------------- softmax (warps 0..3)
    const int r = threadIdx.x;             // row of the tile, also the TMEM lane
    const int q = q0 + r;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m = -INFINITY, l = 0.f, alpha_pending = 0.f;
    float o[D];
#pragma unroll
    for (int i = 0; i < D; ++i) o[i] = 0.f;
    bool ok = true;
    const int hi_key = p.causal ? q + shift : p.S - 1;            // last visible key
    const int lo_key = p.window > 0 ? q + shift - p.window + 1 : 0;  // first visible key
    for (int t = 0; t < n_tiles && ok; ++t) {
      const int s = t & 1;
      const int kv0 = (j_lo + t) * KT;
      ok = warp_all(mbar_wait(&s_full[s], (t >> 1) & 1, abort_flag, st, KID_ATTN_FWD, 6));
      if (!ok) break;
      tc_fence_after();
      // pass 1: row max
      float mx = m;
#pragma unroll 1
      for (int c = 0; c < KT; c += 32) {
        uint32_t v[32];
        tmem_ld_x32(tmem_s + s * 128 + lane_addr + c, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int kv = kv0 + c + i;
          const bool keep = kv < p.S && kv <= hi_key && kv >= lo_key;
          if (keep) mx = fmaxf(mx, __uint_as_float(v[i]) * p.scale_log2);
        }
      }
      const float m_use = mx == -INFINITY ? 0.f : mx;
      const float alpha = m == -INFINITY ? 0.f : exp2f(m - m_use);
      // fold the previous tile's P·V into the accumulator (it frees the P buffer too)
      if (t > 0) {
        ok = warp_all(mbar_wait(pv_full, (t - 1) & 1, abort_flag, st, KID_ATTN_FWD, 7));
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld_x32(tmem_pv + lane_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha_pending + __uint_as_float(v[i]);
        }
      }
      // pass 2: probabilities -> shared memory (swizzled K-major), row sum
      float sum = 0.f;
#pragma unroll 1
      for (int c = 0; c < KT; c += 32) {
        uint32_t v[32];
        tmem_ld_x32(tmem_s + s * 128 + lane_addr + c, v);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float pr[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int kv = kv0 + c + i + e;
            const bool keep = kv < p.S && kv <= hi_key && kv >= lo_key;
            pr[e] = keep ? exp2f(__uint_as_float(v[i + e]) * p.scale_log2 - m_use) : 0.f;
          }
          // the sum uses the values the tensor core will see (rounded to bf16)
          const uint32_t pk = pack_bf16(pr[0], pr[1]);
          const float2 back = unpack_bf16(pk);
          sum += back.x + back.y;
          packed[i >> 1] = pk;
        }
        uint8_t* chunk = sP + (c >> 6) * 16384 + r * 128;
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) {
          const int slot = ((c & 63) >> 3) + sl;
          *reinterpret_cast<uint4*>(chunk + ((slot ^ (r & 7)) << 4)) =
              make_uint4(packed[4 * sl], packed[4 * sl + 1], packed[4 * sl + 2], packed[4 * sl + 3]);
        }
      }
      l = l * alpha + sum;
      m = mx;
      alpha_pending = alpha;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok && n_tiles > 0) {
      ok = warp_all(mbar_wait(pv_full, (n_tiles - 1) & 1, abort_flag, st, KID_ATTN_FWD, 8));
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld_x32(tmem_pv + lane_addr + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[c + i] = o[c + i] * alpha_pending + __uint_as_float(v[i]);
        }
      }
    }
    if (ok && q < p.T) {
      float m_tot = m, scale_o = 1.f;
      if (p.sinks) {
        const float sk = p.sinks[h] * LOG2E;
        m_tot = fmaxf(m, sk);
        const float keep = m == -INFINITY ? 0.f : exp2f(m - m_tot);
        l = l * keep + exp2f(sk - m_tot);
        scale_o = keep;
      }
      const float inv = l > 0.f ? scale_o / l : 0.f;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.o) + (((size_t)b * p.T + q) * p.H + h) * D;
#pragma unroll
      for (int c = 0; c < D; c += 8) {
        uint4 w;
        w.x = pack_bf16(o[c] * inv, o[c + 1] * inv); w.y = pack_bf16(o[c + 2] * inv, o[c + 3] * inv);
        w.z = pack_bf16(o[c + 4] * inv, o[c + 5] * inv); w.w = pack_bf16(o[c + 6] * inv, o[c + 7] * inv);
        *reinterpret_cast<uint4*>(dst + c) = w;
      }
      p.lse[((size_t)b * p.H + h) * p.T + q] = l > 0.f ? (m_tot + log2f(l)) * LN2 : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem_base, Cfg::TMEM_COLS); }
}

template <int D>
static const char* attn_fwd_launch_d(const AttnArgs& a, cudaStream_t stream) {
  using Cfg = AttnFwdCfg<D>;
  AttnFwdParams p;
  const char* err;
  if ((err = make_tmap_2d(&p.tmap_q, a.q, 2, (uint64_t)a.B * a.T, (uint64_t)a.H * D, (uint64_t)a.H * D * 2, 64, QT))) return err;
  if ((err = make_tmap_2d(&p.tmap_kv_k, a.k, 2, (uint64_t)a.B * a.S, (uint64_t)a.G * D, (uint64_t)a.G * D * 2, 64, KT))) return err;
  if ((err = make_tmap_2d(&p.tmap_kv_v, a.v, 2, (uint64_t)a.B * a.S, (uint64_t)a.G * D, (uint64_t)a.G * D * 2, 64, KT))) return err;
  p.o = a.o; p.lse = a.lse; p.sinks = a.sinks; p.status = a.status;
  p.B = a.B; p.T = a.T; p.S = a.S; p.H = a.H; p.G = a.G;
  p.scale_log2 = a.scale * LOG2E; p.causal = a.causal ? 1 : 0; p.window = a.window;
  auto kern = attn_fwd_kernel<D>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES) != cudaSuccess)
      return "cudaFuncSetAttribute(max dynamic shared memory) failed";
    configured = true;
  }
  dim3 grid((a.T + QT - 1) / QT, a.H, a.B);
  kern<<<grid, ATTN_THREADS, Cfg::SMEM_BYTES, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? nullptr : "attention forward launch failed";
}

const char* attn_fwd_launch(const AttnArgs& a, cudaStream_t stream) {
  if (a.H % a.G != 0) return "query heads must be a multiple of key/value heads";
  if (a.D == 128) return attn_fwd_launch_d<128>(a, stream);
  if (a.D == 64) return attn_fwd_launch_d<64>(a, stream);
  return "head_dim must be 64 or 128";
}

}  // namespace bux
