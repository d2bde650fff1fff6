// Softmax attention backward for sm_100a on tcgen05 tensor cores.
//
// Two kernels:
//  * attn_delta_kernel: delta[b,h,t] = sum_d O·dO (and the attention-sink gradient).
//  * attn_bwd_kernel: one CTA per (batch, key/value head, 128-key tile). It keeps K_j
//    and V_j in shared memory and walks every (query head of the group, query tile)
//    that can see the tile, so dK_j and dV_j accumulate in tensor memory across the
//    whole walk and are written once (no atomics, no per-head partials to reduce).
//    Per step, on the tensor core:  S = Q·K^T,  dP = dO·V^T,  then with
//    P = exp(S·scale − lse) and dS = P∘(dP − delta)·scale written to shared memory by
//    the softmax warps:  dV += P^T·dO,  dK += dS^T·Q,  dQ = dS·K. dQ (different key
//    tiles add to the same query rows) is staged in the P / dS buffers once the step's
//    MMAs are done and leaves as TMA reduce-adds of fp32, one per warp and 32 columns.
//    The [rows x 64-column] swizzled tiles that TMA writes serve both as K-major
//    operands (contraction along the head dim) and as MN-major operands (contraction
//    along the rows); only the descriptors differ.
//
// Reference counterparts: FA4's four backward kernels (parallel/fa4.py:431-573) and
// cuDNN's fused backward (parallel/flash.py:573-678).
#include "attention_sm100.h"
#include "common.cuh"
#include "gemm_sm100.h"

namespace bux {

constexpr int KID_ATTN_BWD = 3;
constexpr int BT = 128;
constexpr int BWD_THREADS = 320;  // 8 softmax warps (two per TMEM lane quadrant), TMA warp, MMA warp
constexpr float LOG2E_B = 1.4426950408889634f;

// one warp per (b, t, h) row of D elements
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  const float* __restrict__ lse, const float* __restrict__ sinks,
                                  float* __restrict__ delta, float* __restrict__ dsinks,
                                  int B, int T, int H, int D) {
  const long rows = (long)B * T * H;
  const int lane = threadIdx.x & 31;
  for (long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows;
       row += (long)gridDim.x * (blockDim.x >> 5)) {
    float acc = 0.f;
    for (int i = lane * 2; i < D; i += 64) {
      const float2 a = unpack_bf16(*reinterpret_cast<const uint32_t*>(o + row * D + i));
      const float2 g = unpack_bf16(*reinterpret_cast<const uint32_t*>(d_o + row * D + i));
      acc += a.x * g.x + a.y * g.y;
    }
    acc = warp_sum(acc);
    if (lane == 0) {
      const int h = (int)(row % H);
      const long bt = row / H;
      const int t = (int)(bt % T);
      const int b = (int)(bt / T);
      const size_t idx = ((size_t)b * H + h) * T + t;
      delta[idx] = acc;
      if (sinks && dsinks) atomicAdd(&dsinks[h], -__expf(sinks[h] - lse[idx]) * acc);
    }
  }
}

struct AttnBwdParams {
  alignas(64) CUtensorMap tmap_q;
  alignas(64) CUtensorMap tmap_do;
  alignas(64) CUtensorMap tmap_k;
  alignas(64) CUtensorMap tmap_v;
  alignas(64) CUtensorMap tmap_dq;
  const float* lse; const float* delta;
  const int* row_lo; const int* key_hi;  // documents: see AttnArgs
  float* dq; void* dk; void* dv; Status* status;
  int B, T, S, H, G;
  float scale, scale_log2; int causal, window;
};

template <int D>
struct AttnBwdCfg {
  static constexpr int DC = D / 64;
  static constexpr int TILE_BYTES = DC * 16384;
  static constexpr int PS_BYTES = 2 * 16384;
  static constexpr int SMEM_BYTES = 4 * TILE_BYTES + 2 * PS_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;  // S | dP,dQ | dV | dK  (128 columns each)
};

template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ AttnBwdParams p) {
  using Cfg = AttnBwdCfg<D>;
  constexpr int DC = Cfg::DC;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::TILE_BYTES;
  uint8_t* sQ = sV + Cfg::TILE_BYTES;
  uint8_t* sdO = sQ + Cfg::TILE_BYTES;
  uint8_t* sP = sdO + Cfg::TILE_BYTES;
  uint8_t* sdS = sP + Cfg::PS_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + Cfg::PS_BYTES);
  uint64_t* kv_full = bars;
  uint64_t* qdo_full = bars + 1;
  uint64_t* qdo_empty = bars + 2;
  uint64_t* sdp_full = bars + 3;
  uint64_t* p_ready = bars + 4;
  uint64_t* dq_full = bars + 5;
  uint64_t* dq_done = bars + 6;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 7);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int jt = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  const int kv0 = jt * BT;
  const int shift = p.S - p.T;
  const int n_qt = (p.T + BT - 1) / BT;
  int i_lo = 0, i_hi = n_qt;
  if (p.causal) i_lo = max(0, (kv0 - shift) / BT);
  if (p.window > 0) i_hi = min(n_qt, (kv0 + BT - 1 - shift + p.window - 1) / BT + 1);
  // documents: no query past the end of the tile's last key's document sees the tile
  if (p.key_hi != nullptr) i_hi = min(i_hi, p.key_hi[(size_t)b * p.S + min(kv0 + BT - 1, p.S - 1)] / BT + 1);
  const int per_head = max(0, i_hi - i_lo);
  const int hpg = p.H / p.G;
  const int n_steps = per_head * hpg;
  Status* st = p.status;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1); mbar_init(qdo_full, 1); mbar_init(qdo_empty, 1); mbar_init(sdp_full, 1);
    mbar_init(p_ready, 256); mbar_init(dq_full, 1); mbar_init(dq_done, 256);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;

  if (warp == 8) {
    // -------------------------------------------------------------- TMA producer
    if (elect_one() && n_steps > 0) {
      mbar_expect_tx(kv_full, 2 * Cfg::TILE_BYTES);
      for (int c = 0; c < DC; ++c) {
        tma_load_2d(sK + c * 16384, &p.tmap_k, g * D + c * 64, b * p.S + kv0, kv_full);
        tma_load_2d(sV + c * 16384, &p.tmap_v, g * D + c * 64, b * p.S + kv0, kv_full);
      }
      for (int s = 0; s < n_steps; ++s) {
        if (!mbar_wait(qdo_empty, (s & 1) ^ 1, abort_flag, st, KID_ATTN_BWD, 1)) break;
        const int h = g * hpg + s / per_head;
        const int row = b * p.T + (i_lo + s % per_head) * BT;
        mbar_expect_tx(qdo_full, 2 * Cfg::TILE_BYTES);
        for (int c = 0; c < DC; ++c) {
          tma_load_2d(sQ + c * 16384, &p.tmap_q, h * D + c * 64, row, qdo_full);
          tma_load_2d(sdO + c * 16384, &p.tmap_do, h * D + c * 64, row, qdo_full);
        }
      }
    }
  } else if (warp == 9) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one() && n_steps > 0) {
      const uint32_t id_s = make_idesc(FMT_BF16, FMT_BF16, 128, BT, false, false);
      const uint32_t id_acc = make_idesc(FMT_BF16, FMT_BF16, 128, D, true, true);
      const uint32_t id_dq = make_idesc(FMT_BF16, FMT_BF16, 128, D, false, true);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aDO = smem_u32(sdO);
      const uint32_t aP = smem_u32(sP), aDS = smem_u32(sdS);
      bool ok = mbar_wait(kv_full, 0, abort_flag, st, KID_ATTN_BWD, 2);
      for (int s = 0; s < n_steps && ok; ++s) {
        ok = mbar_wait(qdo_full, s & 1, abort_flag, st, KID_ATTN_BWD, 3);
        if (!ok) break;
        tc_fence_after();
        // S has columns of its own (read before p_ready of the step before): it runs while
        // the previous dQ, which shares dP's columns, is still being drained
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_f16(t_s, make_smem_desc(aQ + off, 0, 1024, 2), make_smem_desc(aK + off, 0, 1024, 2), id_s, kk > 0);
        }
        if (s > 0) ok = mbar_wait(dq_done, (s - 1) & 1, abort_flag, st, KID_ATTN_BWD, 4);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_f16(t_dp, make_smem_desc(aDO + off, 0, 1024, 2), make_smem_desc(aV + off, 0, 1024, 2), id_s, kk > 0);
        }
        tc_commit(sdp_full);
        ok = mbar_wait(p_ready, s & 1, abort_flag, st, KID_ATTN_BWD, 5);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk) {  // contraction over the 128 query rows
          const uint64_t pa = make_smem_desc(aP + kk * 2048, 16384, 1024, 2);
          const uint64_t dsa = make_smem_desc(aDS + kk * 2048, 16384, 1024, 2);
          const uint64_t dob = make_smem_desc(aDO + kk * 2048, 16384, 1024, 2);
          const uint64_t qb = make_smem_desc(aQ + kk * 2048, 16384, 1024, 2);
          mma_f16(t_dv, pa, dob, id_acc, (s > 0 || kk > 0) ? 1u : 0u);
          mma_f16(t_dk, dsa, qb, id_acc, (s > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk) {  // contraction over the 128 keys
          const uint64_t dsa = make_smem_desc(aDS + (kk >> 2) * 16384 + (kk & 3) * 32, 0, 1024, 2);
          const uint64_t kb = make_smem_desc(aK + kk * 2048, 16384, 1024, 2);
          mma_f16(t_dp, dsa, kb, id_dq, kk > 0);
        }
        tc_commit(dq_full);
        tc_commit(qdo_empty);
      }
    }
  } else {
    // -------------------------------------------------------------- softmax / drain warps
    // Two warps share each 32-lane quadrant of tensor memory: warps 0-3 take the first 64
    // columns of S / dP, warps 4-7 the other 64, so each scheduler has two warps to
    // interleave and the exp / dS chain per step is half as long.
    const int r = threadIdx.x & 127, lane = threadIdx.x & 31, half = warp >> 2;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    bool ok = true;
    for (int s = 0; s < n_steps && ok; ++s) {
      const int h = g * hpg + s / per_head;
      const int q = (i_lo + s % per_head) * BT + r;
      const bool row_ok = q < p.T;
      const size_t stat = ((size_t)b * p.H + h) * p.T + (row_ok ? q : 0);
      const float lse2 = row_ok ? p.lse[stat] * LOG2E_B : 0.f;
      const float dlt = row_ok ? p.delta[stat] : 0.f;
      const int hi_key = p.causal ? q + shift : p.S - 1;
      int lo_key = p.window > 0 ? q + shift - p.window + 1 : 0;
      if (p.row_lo != nullptr && row_ok) lo_key = max(lo_key, p.row_lo[(size_t)b * p.T + q]);
      ok = warp_all(mbar_wait(sdp_full, s & 1, abort_flag, st, KID_ATTN_BWD, 6));
      if (!ok) break;
      tc_fence_after();
      // the dQ tile of the previous step was staged where P and dS go: its reduction must
      // have read this warp's rows before they are overwritten
      if (lane == 0) tma_store_wait_read();
      __syncwarp();
      const bool full_row = row_ok && kv0 + BT - 1 <= hi_key && kv0 >= lo_key && kv0 + BT <= p.S && lse2 > -INFINITY;
      const bool any_row = row_ok && lse2 > -INFINITY;
      const int c_first = half * 64;
      const float nlse2 = -lse2, ndlt = -dlt * p.scale;
#pragma unroll 1
      for (int ci = 0; ci < 2; ++ci) {
        const int c = c_first + ci * 32;
        uint32_t cs[32], cd[32];
        tmem_ld_x32(t_s + lane_addr + c, cs);
        tmem_ld_x32(t_dp + lane_addr + c, cd);
        tmem_ld_wait();
        uint32_t pp[16], ds[16];
        if (full_row) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            // P = 2^(s·scale·log2e − lse·log2e); dS = P·(dP·scale − delta·scale)
            const float p0 = ex2_approx(fmaf(__uint_as_float(cs[i]), p.scale_log2, nlse2));
            const float p1 = ex2_approx(fmaf(__uint_as_float(cs[i + 1]), p.scale_log2, nlse2));
            pp[i >> 1] = pack_bf16(p0, p1);
            ds[i >> 1] = pack_bf16(p0 * fmaf(__uint_as_float(cd[i]), p.scale, ndlt),
                                   p1 * fmaf(__uint_as_float(cd[i + 1]), p.scale, ndlt));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            float pr[2], dr[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int kv = kv0 + c + i + e;
              const bool keep = any_row && kv < p.S && kv <= hi_key && kv >= lo_key;
              pr[e] = keep ? ex2_approx(fmaf(__uint_as_float(cs[i + e]), p.scale_log2, nlse2)) : 0.f;
              dr[e] = pr[e] * fmaf(__uint_as_float(cd[i + e]), p.scale, ndlt);
            }
            pp[i >> 1] = pack_bf16(pr[0], pr[1]);
            ds[i >> 1] = pack_bf16(dr[0], dr[1]);
          }
        }
        const int base = half * 16384 + r * 128;
#pragma unroll
        for (int sl = 0; sl < 4; ++sl) {
          const int slot = ((ci << 2) + sl) ^ (r & 7);
          *reinterpret_cast<uint4*>(sP + base + (slot << 4)) = make_uint4(pp[4 * sl], pp[4 * sl + 1], pp[4 * sl + 2], pp[4 * sl + 3]);
          *reinterpret_cast<uint4*>(sdS + base + (slot << 4)) = make_uint4(ds[4 * sl], ds[4 * sl + 1], ds[4 * sl + 2], ds[4 * sl + 3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(p_ready);
      // dQ of this step: tensor memory -> this warp's rows of the staging tiles (the P / dS
      // buffers, free once the step's MMAs have completed) -> one reduce-add per 32 columns
      ok = warp_all(mbar_wait(dq_full, s & 1, abort_flag, st, KID_ATTN_BWD, 7));
      if (!ok) break;
      tc_fence_after();
      // This warp stages the 32-column chunks half, half+2, ... of its 32 rows: the
      // same shared-memory rows it writes P and dS to, so every hazard on the staging
      // tiles stays inside the warp.
      {
        uint32_t v[D / 64][32];
#pragma unroll
        for (int j = 0; j < D / 64; ++j) tmem_ld_x32(t_dp + lane_addr + (half + 2 * j) * 32, v[j]);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < D / 64; ++j) {
          uint8_t* dst = sP + (half + 2 * j) * 16384 + r * 128;
#pragma unroll
          for (int sl = 0; sl < 8; ++sl)
            *reinterpret_cast<uint4*>(dst + ((sl ^ (r & 7)) << 4)) =
                make_uint4(v[j][4 * sl], v[j][4 * sl + 1], v[j][4 * sl + 2], v[j][4 * sl + 3]);
        }
      }
      tc_fence_before();
      mbar_arrive(dq_done);
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        const int row0 = b * p.T + (i_lo + s % per_head) * BT + (warp & 3) * 32;
#pragma unroll
        for (int j = 0; j < D / 64; ++j) {
          const int ci = half + 2 * j;
          tma_reduce_add_2d(&p.tmap_dq, sP + ci * 16384 + (warp & 3) * 4096, h * D + ci * 32, row0);
        }
        tma_store_commit();
      }
    }
    if (lane == 0) tma_store_wait_all();
    __syncwarp();
    // dK / dV of this key tile: complete once the last step's MMAs have (dq_full waited above)
    // tcgen05.ld is warp-collective: every thread of the warp takes part, only the
    // stores are masked.
    const int kv = kv0 + r;
    const bool store = ok && kv < p.S;
    const bool all_ok = __all_sync(0xffffffffu, ok);
    {
      __nv_bfloat16* dkrow = reinterpret_cast<__nv_bfloat16*>(p.dk) + (((size_t)b * p.S + (store ? kv : 0)) * p.G + g) * D;
      __nv_bfloat16* dvrow = reinterpret_cast<__nv_bfloat16*>(p.dv) + (((size_t)b * p.S + (store ? kv : 0)) * p.G + g) * D;
#pragma unroll 1
      for (int c = half * (D / 2); c < (half + 1) * (D / 2); c += 32) {
        uint32_t a[32], bb[32];
        if (n_steps > 0 && all_ok) {
          tmem_ld_x32(t_dk + lane_addr + c, a);
          tmem_ld_x32(t_dv + lane_addr + c, bb);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) { a[i] = 0; bb[i] = 0; }
        }
        if (!store) continue;
#pragma unroll
        for (int i = 0; i < 32; i += 8) {
          uint4 x, y;
          x.x = pack_bf16(__uint_as_float(a[i]), __uint_as_float(a[i + 1])); x.y = pack_bf16(__uint_as_float(a[i + 2]), __uint_as_float(a[i + 3]));
          x.z = pack_bf16(__uint_as_float(a[i + 4]), __uint_as_float(a[i + 5])); x.w = pack_bf16(__uint_as_float(a[i + 6]), __uint_as_float(a[i + 7]));
          y.x = pack_bf16(__uint_as_float(bb[i]), __uint_as_float(bb[i + 1])); y.y = pack_bf16(__uint_as_float(bb[i + 2]), __uint_as_float(bb[i + 3]));
          y.z = pack_bf16(__uint_as_float(bb[i + 4]), __uint_as_float(bb[i + 5])); y.w = pack_bf16(__uint_as_float(bb[i + 6]), __uint_as_float(bb[i + 7]));
          *reinterpret_cast<uint4*>(dkrow + c + i) = x;
          *reinterpret_cast<uint4*>(dvrow + c + i) = y;
        }
      }
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
static const char* attn_bwd_launch_d(const AttnArgs& a, cudaStream_t stream) {
  using Cfg = AttnBwdCfg<D>;
  AttnBwdParams p;
  const char* err;
  const uint64_t qw = (uint64_t)a.H * D, kw = (uint64_t)a.G * D;
  if ((err = make_tmap_2d(&p.tmap_q, a.q, 2, (uint64_t)a.B * a.T, qw, qw * 2, 64, BT))) return err;
  if ((err = make_tmap_2d(&p.tmap_do, a.d_o, 2, (uint64_t)a.B * a.T, qw, qw * 2, 64, BT))) return err;
  if ((err = make_tmap_2d(&p.tmap_k, a.k, 2, (uint64_t)a.B * a.S, kw, kw * 2, 64, BT))) return err;
  if ((err = make_tmap_2d(&p.tmap_v, a.v, 2, (uint64_t)a.B * a.S, kw, kw * 2, 64, BT))) return err;
  if ((err = make_tmap_2d(&p.tmap_dq, a.dq, 4, (uint64_t)a.B * a.T, qw, qw * 4, 32, 32))) return err;
  p.row_lo = a.row_lo; p.key_hi = a.key_hi;
  p.lse = a.lse; p.delta = a.delta; p.dq = reinterpret_cast<float*>(a.dq); p.dk = a.dk; p.dv = a.dv;
  p.status = a.status;
  p.B = a.B; p.T = a.T; p.S = a.S; p.H = a.H; p.G = a.G;
  p.scale = a.scale; p.scale_log2 = a.scale * LOG2E_B; p.causal = a.causal ? 1 : 0; p.window = a.window;
  auto kern = attn_bwd_kernel<D>;
  static bool configured[64] = {};
  if (!allow_dynamic_smem(kern, Cfg::SMEM_BYTES, configured))
    return "cudaFuncSetAttribute(max dynamic shared memory) failed";
  const long rows = (long)a.B * a.T * a.H;
  attn_delta_kernel<<<(int)min((rows + 7) / 8, 148L * 16), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(a.o), reinterpret_cast<const __nv_bfloat16*>(a.d_o), a.lse,
      a.sinks, a.delta, a.dsinks, a.B, a.T, a.H, D);
  dim3 grid((a.S + BT - 1) / BT, a.G, a.B);
  kern<<<grid, BWD_THREADS, Cfg::SMEM_BYTES, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? nullptr : "attention backward launch failed";
}

const char* attn_bwd_launch(const AttnArgs& a, cudaStream_t stream) {
  if (a.H % a.G != 0) return "query heads must be a multiple of key/value heads";
  if (a.D == 128) return attn_bwd_launch_d<128>(a, stream);
  if (a.D == 64) return attn_bwd_launch_d<64>(a, stream);
  return "head_dim must be 64 or 128";
}

}  // namespace bux
