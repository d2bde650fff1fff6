// Softmax attention for sm_100a on tcgen05 tensor cores, forward pass.
//
// One CTA per (batch, query head, pair of 128-query tiles); 320 threads:
//   warps 0..7  two softmax warpgroups, one per query tile, one query row per thread.
//               Each reads S = Q·K^T from tensor memory (tcgen05.ld), turns it into
//               P = exp2(S·scale - ref) in one pass against a per-row reference that
//               only moves when a row max outgrows it by 2^64 (then O in tensor memory
//               and the running sum are rescaled), and writes P (bf16) into shared
//               memory in the tensor core's swizzled K-major layout.
//   warp 8      TMA producer: both Q tiles once, then K (2 stages) and V tiles (plain
//               TMA loads, no multicast).
//   warp 9      MMA issuer: S_x(j) = Q_x·K_j^T and O_x += P_x(j)·V_j, accumulated in
//               tensor memory; the two tiles' MMAs interleave so the tensor core works
//               on one tile while the other tile's softmax runs.
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
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

struct AttnFwdParams {
  alignas(64) CUtensorMap tmap_q;
  alignas(64) CUtensorMap tmap_kv_k;
  alignas(64) CUtensorMap tmap_kv_v;
  void* o; float* lse; const float* sinks; Status* status;
  const int* row_lo;  // [B, T] first visible key of each query (documents), or null
  int B, T, S, H, G;
  float scale_log2; int causal, window;
};

// Two 128-query tiles per CTA, one softmax warpgroup each, so that the tensor core
// works on one tile while the other tile's softmax runs.
constexpr int FWD_THREADS = 320;          // 8 softmax warps + TMA warp + MMA warp
constexpr float RESCALE_THRESHOLD = 64.f; // log2 units a row max may outgrow its reference

template <int D>
struct AttnFwdCfg {
  static constexpr int DC = D / 64;
  static constexpr int TILE_BYTES = DC * 16384;   // one [128 x D] bf16 tile
  static constexpr int P_BYTES = 2 * 16384;       // [128 x 128] bf16
  static constexpr int V_STAGES = D == 128 ? 1 : 2;
  static constexpr int SMEM_BYTES = TILE_BYTES * (2 + 2 + V_STAGES) + 2 * P_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;           // S_A, S_B (128 each), O_A, O_B (D each)
};

template <int D>
__global__ void __launch_bounds__(FWD_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ AttnFwdParams p) {
  using Cfg = AttnFwdCfg<D>;
  constexpr int DC = Cfg::DC;
  constexpr int VS = Cfg::V_STAGES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                               // 2 tiles
  uint8_t* sK = sQ + 2 * Cfg::TILE_BYTES;           // 2 stages
  uint8_t* sV = sK + 2 * Cfg::TILE_BYTES;           // VS stages
  uint8_t* sP = sV + VS * Cfg::TILE_BYTES;          // 2 tiles
  uint64_t* bars = reinterpret_cast<uint64_t*>(sP + 2 * Cfg::P_BYTES);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* k_empty = bars + 3;    // [2]
  uint64_t* v_full = bars + 5;     // [2]
  uint64_t* v_empty = bars + 7;    // [2]
  uint64_t* s_full = bars + 9;     // [2] per query tile
  uint64_t* p_ready = bars + 11;   // [2]
  uint64_t* pv_full = bars + 13;   // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int n_qt = (p.T + 2 * QT - 1) / (2 * QT);
  const int qt = n_qt - 1 - blockIdx.x;  // long (late) rows first under a causal mask
  const int h = blockIdx.y, b = blockIdx.z;
  const int g = h / (p.H / p.G);
  const int q0 = qt * 2 * QT;
  const int shift = p.S - p.T;
  const int s_tiles = (p.S + KT - 1) / KT;
  int lo[2], hi[2];
#pragma unroll
  for (int x = 0; x < 2; ++x) {
    const int qx = q0 + x * QT;
    hi[x] = s_tiles;
    if (p.causal) hi[x] = min(hi[x], (qx + QT - 1 + shift) / KT + 1);
    lo[x] = p.window > 0 ? max(0, (qx + shift - p.window + 1) / KT) : 0;
    // documents: the tile's first query has the earliest document start of the tile
    if (p.row_lo != nullptr && qx < p.T) lo[x] = max(lo[x], p.row_lo[(size_t)b * p.T + qx] / KT);
    if (qx >= p.T || hi[x] <= lo[x]) { lo[x] = 0; hi[x] = 0; }
  }
  const bool any0 = hi[0] > lo[0], any1 = hi[1] > lo[1];
  const int j_lo = any0 && any1 ? min(lo[0], lo[1]) : (any0 ? lo[0] : lo[1]);
  const int j_hi = max(hi[0], hi[1]);
  // With documents the second query tile may start seeing keys after the first one's last
  // key tile: the key tiles in between are seen by neither and are not loaded. Tiles that
  // are loaded are numbered 0, 1, ... (`slot_of`) for the stage rings and their parities.
  const int gap_at = (any0 && any1 && lo[1] > hi[0]) ? hi[0] : j_hi;
  const int gap = (any0 && any1 && lo[1] > hi[0]) ? lo[1] - hi[0] : 0;
  const int n_tiles = (any0 || any1) ? j_hi - j_lo - gap : 0;
  auto slot_of = [&](int j) { return j - j_lo - (j >= gap_at ? gap : 0); };
  auto tile_of = [&](int t) { return j_lo + t + (j_lo + t >= gap_at ? gap : 0); };
  Status* st = p.status;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_ready[i], 128); mbar_init(&pv_full[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // -------------------------------------------------------------- TMA producer
    if (elect_one() && n_tiles > 0) {
      mbar_expect_tx(q_full, 2 * Cfg::TILE_BYTES);
      for (int x = 0; x < 2; ++x)
        for (int c = 0; c < DC; ++c)
          tma_load_2d(sQ + x * Cfg::TILE_BYTES + c * 16384, &p.tmap_q, h * D + c * 64, b * p.T + q0 + x * QT, q_full);
      for (int t = 0; t < n_tiles; ++t) {
        const int row = b * p.S + tile_of(t) * KT;
        const int ks = t & 1, vs = t % VS;
        if (!mbar_wait(&k_empty[ks], ((t >> 1) & 1) ^ 1, abort_flag, st, KID_ATTN_FWD, 1)) break;
        mbar_expect_tx(&k_full[ks], Cfg::TILE_BYTES);
        for (int c = 0; c < DC; ++c)
          tma_load_2d(sK + ks * Cfg::TILE_BYTES + c * 16384, &p.tmap_kv_k, g * D + c * 64, row, &k_full[ks]);
        if (!mbar_wait(&v_empty[vs], ((t / VS) & 1) ^ 1, abort_flag, st, KID_ATTN_FWD, 2)) break;
        mbar_expect_tx(&v_full[vs], Cfg::TILE_BYTES);
        for (int c = 0; c < DC; ++c)
          tma_load_2d(sV + vs * Cfg::TILE_BYTES + c * 16384, &p.tmap_kv_v, g * D + c * 64, row, &v_full[vs]);
      }
    }
  } else if (warp == 9) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one() && n_tiles > 0) {
      const uint32_t idesc_s = make_idesc(FMT_BF16, FMT_BF16, 128, KT, false, false);
      const uint32_t idesc_pv = make_idesc(FMT_BF16, FMT_BF16, 128, D, false, true);
      bool ok = true;
      auto active = [&](int x, int j) { return j >= lo[x] && j < hi[x]; };
      int next_s[2] = {lo[0], lo[1]};  // next key tile whose S_x has not been issued
      // S_x(j) = Q_x · K_j^T ; frees K_j when x is its last user
      auto issue_s = [&](int x, int j) {
        const int t = slot_of(j), ks = t & 1;
        if (!mbar_wait(&k_full[ks], (t >> 1) & 1, abort_flag, st, KID_ATTN_FWD, 3)) { ok = false; return; }
        tc_fence_after();
        const uint32_t a0 = smem_u32(sQ + x * Cfg::TILE_BYTES), b0 = smem_u32(sK + ks * Cfg::TILE_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_f16(tmem_base + x * 128, make_smem_desc(a0 + off, 0, 1024, 2), make_smem_desc(b0 + off, 0, 1024, 2), idesc_s, kk > 0);
        }
        tc_commit(&s_full[x]);
        next_s[x] = j + 1;
        // K_j is free once every query tile that uses it has issued its S_x(j)
        const int other = x ^ 1;
        if (!active(other, j) || next_s[other] > j) tc_commit(&k_empty[ks]);
      };
      ok = mbar_wait(q_full, 0, abort_flag, st, KID_ATTN_FWD, 4);
      int done[2] = {0, 0};  // tiles processed per query tile (for barrier parities)
      // a query tile's first S is issued when the walk reaches its first key tile (at once for
      // the tile that starts the walk): issuing it earlier would wait for a key tile that the
      // two-stage ring cannot hold yet
      for (int x = 0; x < 2 && ok; ++x)
        if (hi[x] > lo[x] && lo[x] == j_lo) issue_s(x, lo[x]);
      for (int j = j_lo; j < j_hi && ok; ++j) {
        if (j >= gap_at && j < gap_at + gap) continue;
        const int t = slot_of(j), vs = t % VS;
        for (int x = 0; x < 2 && ok; ++x)
          if (hi[x] > lo[x] && lo[x] == j && next_s[x] == j && j != j_lo) issue_s(x, j);
        for (int x = 0; x < 2 && ok; ++x) {
          if (!active(x, j)) continue;
          ok = mbar_wait(&p_ready[x], done[x] & 1, abort_flag, st, KID_ATTN_FWD, 5);
          if (!ok) break;
          ok = mbar_wait(&v_full[vs], (t / VS) & 1, abort_flag, st, KID_ATTN_FWD, 6);
          if (!ok) break;
          tc_fence_after();
          const uint32_t a0 = smem_u32(sP + x * Cfg::P_BYTES), b0 = smem_u32(sV + vs * Cfg::TILE_BYTES);
#pragma unroll
          for (int kk = 0; kk < KT / 16; ++kk) {
            const uint64_t ad = make_smem_desc(a0 + (kk >> 2) * 16384 + (kk & 3) * 32, 0, 1024, 2);
            const uint64_t bd = make_smem_desc(b0 + kk * 2048, 16384, 1024, 2);
            mma_f16(tmem_base + 256 + x * 128, ad, bd, idesc_pv, (j > lo[x] || kk > 0) ? 1u : 0u);
          }
          tc_commit(&pv_full[x]);
          if (x == 1 || !active(1, j)) tc_commit(&v_empty[vs]);
          ++done[x];
          if (j + 1 < hi[x]) issue_s(x, j + 1);
        }
      }
    }
  } else {
    // -------------------------------------------------------------- softmax warpgroups
    const int x = warp >> 2;                 // which query tile
    const int r = threadIdx.x & 127;         // row of the tile = TMEM lane
    const int q = q0 + x * QT + r;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + x * 128 + lane_addr;
    const uint32_t t_o = tmem_base + 256 + x * 128 + lane_addr;
    uint8_t* myP = sP + x * Cfg::P_BYTES;
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    const int hi_key = p.causal ? q + shift : p.S - 1;
    int lo_key = p.window > 0 ? q + shift - p.window + 1 : 0;
    if (p.row_lo != nullptr && q < p.T) lo_key = max(lo_key, p.row_lo[(size_t)b * p.T + q]);
    int done = 0;
    for (int j = lo[x]; j < hi[x] && ok; ++j, ++done) {
      const int kv0 = j * KT;
      ok = warp_all(mbar_wait(&s_full[x], done & 1, abort_flag, st, KID_ATTN_FWD, 7));
      if (!ok) break;
      tc_fence_after();
      // S_j complete implies P·V of tile j-1 complete (same issue queue): O may be touched.
      // tcgen05.ld is warp-collective, so the whole warp takes this branch together
      if (__any_sync(0xffffffffu, m_ref == -INFINITY)) {
        // first tile with a visible key: find the row max to use as the reference
        float mx = -INFINITY;
#pragma unroll 1
        for (int c = 0; c < KT; c += 32) {
          uint32_t v[32];
          tmem_ld_x32(t_s + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kv = kv0 + c + i;
            if (kv < p.S && kv <= hi_key && kv >= lo_key) mx = fmaxf(mx, __uint_as_float(v[i]) * p.scale_log2);
          }
        }
        if (m_ref == -INFINITY) m_ref = mx;
      }
      // rows whose whole tile is visible skip the per-element mask
      const bool full_row = kv0 + KT - 1 <= hi_key && kv0 >= lo_key && kv0 + KT <= p.S;
      for (int attempt = 0; attempt < 2; ++attempt) {
        float sum = 0.f, sum1 = 0.f, mx = -INFINITY, mx_raw = -INFINITY;
        const float ref = m_ref == -INFINITY ? 0.f : m_ref;
        const float nref = -ref, sc = p.scale_log2;
        uint32_t v[2][32];
        tmem_ld_x32(t_s, v[0]);
#pragma unroll
        for (int ci = 0; ci < KT / 32; ++ci) {
          const int c = ci * 32;
          tmem_ld_wait();
          // the next chunk's load runs while this one is turned into probabilities
          if (ci + 1 < KT / 32) tmem_ld_x32(t_s + c + 32, v[(ci + 1) & 1]);
          const uint32_t(&cur)[32] = v[ci & 1];
          uint32_t packed[16];
          if (full_row) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              // per element: one max on the raw score, one fused multiply-add, one ex2, one add
              const float x0 = __uint_as_float(cur[i]), x1 = __uint_as_float(cur[i + 1]);
              mx_raw = fmaxf(mx_raw, fmaxf(x0, x1));
              const float p0 = ex2_approx(fmaf(x0, sc, nref)), p1 = ex2_approx(fmaf(x1, sc, nref));
              sum += p0;
              sum1 += p1;
              packed[i >> 1] = pack_bf16(p0, p1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float pr[2];
#pragma unroll
              for (int e = 0; e < 2; ++e) {
                const int kv = kv0 + c + i + e;
                const bool keep = kv < p.S && kv <= hi_key && kv >= lo_key;
                const float xv = __uint_as_float(cur[i + e]);
                if (keep) mx_raw = fmaxf(mx_raw, xv);
                pr[e] = keep ? ex2_approx(fmaf(xv, sc, nref)) : 0.f;
              }
              sum += pr[0] + pr[1];
              packed[i >> 1] = pack_bf16(pr[0], pr[1]);
            }
          }
          uint8_t* chunk = myP + (c >> 6) * 16384 + r * 128;
#pragma unroll
          for (int sl = 0; sl < 4; ++sl) {
            const int slot = ((c & 63) >> 3) + sl;
            *reinterpret_cast<uint4*>(chunk + ((slot ^ (r & 7)) << 4)) =
                make_uint4(packed[4 * sl], packed[4 * sl + 1], packed[4 * sl + 2], packed[4 * sl + 3]);
          }
        }
        sum += sum1;
        mx = mx_raw * sc;  // the scale is positive: the max of the scaled scores
        // The reference only moves when a row max outgrows it by a wide margin: P and the
        // running sums stay exact relative to the reference, so this is rare.
        const bool redo = mx > m_ref + RESCALE_THRESHOLD;
        if (!__any_sync(0xffffffffu, redo) || attempt == 1) { l += sum; break; }
        // rescale what was accumulated so far to the new reference, then redo this tile
        const float alpha = redo ? exp2f(m_ref - mx) : 1.f;
        if (done > 0) {
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t v[32];
            tmem_ld_x32(t_o + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_x32(t_o + c, v);
          }
          tmem_st_wait();
        }
        l *= alpha;
        if (redo) m_ref = mx;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&p_ready[x]);
    }
    float ov[D];
    if (done > 0 && ok) {
      ok = warp_all(mbar_wait(&pv_full[x], (done - 1) & 1, abort_flag, st, KID_ATTN_FWD, 8));
      if (ok) {
        tc_fence_after();
#pragma unroll
        for (int c = 0; c < D; c += 32) {
          uint32_t v[32];
          tmem_ld_x32(t_o + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[c + i] = __uint_as_float(v[i]);
        }
      }
    } else {
#pragma unroll
      for (int i = 0; i < D; ++i) ov[i] = 0.f;
    }
    if (ok && q < p.T) {
      float m_tot = m_ref, scale_o = 1.f;
      if (p.sinks) {
        const float sk = p.sinks[h] * LOG2E;
        m_tot = fmaxf(m_ref, sk);
        const float keep = m_ref == -INFINITY ? 0.f : exp2f(m_ref - m_tot);
        l = l * keep + exp2f(sk - m_tot);
        scale_o = keep;
      }
      const float inv = l > 0.f ? scale_o / l : 0.f;
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.o) + (((size_t)b * p.T + q) * p.H + h) * D;
#pragma unroll
      for (int c = 0; c < D; c += 8) {
        uint4 w;
        w.x = pack_bf16(ov[c] * inv, ov[c + 1] * inv); w.y = pack_bf16(ov[c + 2] * inv, ov[c + 3] * inv);
        w.z = pack_bf16(ov[c + 4] * inv, ov[c + 5] * inv); w.w = pack_bf16(ov[c + 6] * inv, ov[c + 7] * inv);
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
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, Cfg::TMEM_COLS); }
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
  p.row_lo = a.row_lo;
  p.B = a.B; p.T = a.T; p.S = a.S; p.H = a.H; p.G = a.G;
  p.scale_log2 = a.scale * LOG2E; p.causal = a.causal ? 1 : 0; p.window = a.window;
  auto kern = attn_fwd_kernel<D>;
  static bool configured[64] = {};
  if (!allow_dynamic_smem(kern, Cfg::SMEM_BYTES, configured))
    return "cudaFuncSetAttribute(max dynamic shared memory) failed";
  dim3 grid((a.T + 2 * QT - 1) / (2 * QT), a.H, a.B);
  kern<<<grid, FWD_THREADS, Cfg::SMEM_BYTES, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? nullptr : "attention forward launch failed";
}

const char* attn_fwd_launch(const AttnArgs& a, cudaStream_t stream) {
  if (a.H % a.G != 0) return "query heads must be a multiple of key/value heads";
  if (a.D == 128) return attn_fwd_launch_d<128>(a, stream);
  if (a.D == 64) return attn_fwd_launch_d<64>(a, stream);
  return "head_dim must be 64 or 128";
}

}  // namespace bux
