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
  float* dq; void* dk; void* dv; Status* status; unsigned int* phase_cycles;
  int B, T, S, H, G;
  float scale, scale_log2; int causal, window;
};

template <int D>
struct AttnBwdCfg {
  static constexpr int DC = D / 64;
  static constexpr int TILE_BYTES = DC * 16384;
  static constexpr int PS_BYTES = 2 * 16384;
  // K, V, two Q buffers, dO, P, dS
  static constexpr int SMEM_BYTES = 5 * TILE_BYTES + 2 * PS_BYTES + 1024 + 256;
  static constexpr int TMEM_COLS = 512;  // S | dP,dQ | dV | dK  (128 columns each)
};

// Barrier slots (one 8-byte word each).
enum BwdBar {
  B_KV_FULL = 0, B_Q_FULL0, B_Q_FULL1, B_Q_FREE0, B_Q_FREE1, B_DO_FULL, B_DO_FREE, B_S_FULL, B_S_READ,
  B_DP_FULL, B_PDS_READY, B_DQ_FULL, B_DQ_DONE, B_COUNT
};

// Schedule. Step s pairs the key tile with one (query head, query tile).
//
//   tensor core, step s:  dV += P(s)^T·dO | dQ(s) = dS·K | dK += dS^T·Q(s) | dP(s+1) = dO·V^T | S(s+2) = Q·K^T
//   softmax warps:        P(s+1) from S(s+1), kept in registers while the step's MMAs run;
//                         dQ(s) out of tensor memory into the P and dS tiles (free once dV and dK
//                         have run), TMA reduce-adds of fp32 from both; dS(s+1) from dP(s+1) while
//                         those reduces read shared memory; then P(s+1) and dS(s+1) are stored
//                         over the staged halves and the next step's MMAs start.
//
// Q has two buffers (S runs two steps ahead of dK), dO one (it is free after dV, the step's first
// MMA). dQ shares dP's columns of tensor memory: dP(s+1) is issued once the warps have read dQ(s).
template <int D>
__global__ void __launch_bounds__(BWD_THREADS, 1)
attn_bwd_kernel(const __grid_constant__ AttnBwdParams p) {
  using Cfg = AttnBwdCfg<D>;
  constexpr int DC = Cfg::DC;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + Cfg::TILE_BYTES;
  uint8_t* sQ = sV + Cfg::TILE_BYTES;          // two buffers
  uint8_t* sdO = sQ + 2 * Cfg::TILE_BYTES;
  uint8_t* sP = sdO + Cfg::TILE_BYTES;
  uint8_t* sdS = sP + Cfg::PS_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + Cfg::PS_BYTES);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + B_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  unsigned int* phase = reinterpret_cast<unsigned int*>(bars + B_COUNT + 1);   // 32 counters

  const int warp = threadIdx.x >> 5;
  const int jt = blockIdx.x, g = blockIdx.y, b = blockIdx.z;
  // phase timers: one thread of softmax warp 0 and the MMA issuer of the first CTA add the
  // cycles since their last mark to a counter in shared memory
  const bool timed = p.phase_cycles != nullptr && (blockIdx.x | blockIdx.y | blockIdx.z) == 0 &&
                     (threadIdx.x == 0 || warp == 9);
  unsigned int t_mark = timed ? (unsigned int)clock64() : 0u;
#define BWD_MARK(slot)                                     \
  if (timed) {                                             \
    const unsigned int t_now = (unsigned int)clock64();    \
    atomicAdd(&phase[(slot)], t_now - t_mark);             \
    t_mark = t_now;                                        \
  }
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
    mbar_init(bars + B_KV_FULL, 1);
    mbar_init(bars + B_Q_FULL0, 1); mbar_init(bars + B_Q_FULL1, 1);
    mbar_init(bars + B_Q_FREE0, 1); mbar_init(bars + B_Q_FREE1, 1);
    mbar_init(bars + B_DO_FULL, 1); mbar_init(bars + B_DO_FREE, 1);
    mbar_init(bars + B_S_FULL, 1); mbar_init(bars + B_S_READ, 256);
    mbar_init(bars + B_DP_FULL, 1); mbar_init(bars + B_PDS_READY, 256);
    mbar_init(bars + B_DQ_FULL, 1); mbar_init(bars + B_DQ_DONE, 256);
    *abort_flag = 0;
    for (int i = 0; i < 32; ++i) phase[i] = 0;
    mbar_fence_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_s = tmem_base, t_dp = tmem_base + 128, t_dv = tmem_base + 256, t_dk = tmem_base + 384;
#define BWD_WAIT(slot, parity, site) mbar_wait(bars + (slot), (parity), abort_flag, st, KID_ATTN_BWD, (site))

  if (warp == 8) {
    // -------------------------------------------------------------- TMA producer
    if (elect_one() && n_steps > 0) {
      auto load_q = [&](int s) {
        const int h = g * hpg + s / per_head;
        const int row = b * p.T + (i_lo + s % per_head) * BT;
        uint64_t* full = bars + B_Q_FULL0 + (s & 1);
        mbar_expect_tx(full, Cfg::TILE_BYTES);
        for (int c = 0; c < DC; ++c)
          tma_load_2d(sQ + (s & 1) * Cfg::TILE_BYTES + c * 16384, &p.tmap_q, h * D + c * 64, row, full);
      };
      auto load_do = [&](int s) {
        const int h = g * hpg + s / per_head;
        const int row = b * p.T + (i_lo + s % per_head) * BT;
        mbar_expect_tx(bars + B_DO_FULL, Cfg::TILE_BYTES);
        for (int c = 0; c < DC; ++c) tma_load_2d(sdO + c * 16384, &p.tmap_do, h * D + c * 64, row, bars + B_DO_FULL);
      };
      mbar_expect_tx(bars + B_KV_FULL, 2 * Cfg::TILE_BYTES);
      for (int c = 0; c < DC; ++c) {
        tma_load_2d(sK + c * 16384, &p.tmap_k, g * D + c * 64, b * p.S + kv0, bars + B_KV_FULL);
        tma_load_2d(sV + c * 16384, &p.tmap_v, g * D + c * 64, b * p.S + kv0, bars + B_KV_FULL);
      }
      load_q(0);
      load_do(0);
      if (n_steps > 1) load_q(1);
      for (int s = 0; s < n_steps; ++s) {
        // dO(s+1) once dP(s) and dV(s) have read dO(s); Q(s+2) once dK(s) has read Q(s)
        if (s + 1 < n_steps) {
          if (!BWD_WAIT(B_DO_FREE, s & 1, 1)) break;
          load_do(s + 1);
        }
        if (s + 2 < n_steps) {
          if (!BWD_WAIT(B_Q_FREE0 + (s & 1), (s >> 1) & 1, 2)) break;
          load_q(s + 2);
        }
      }
    }
  } else if (warp == 9) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one() && n_steps > 0) {
      const uint32_t id_s = make_idesc(FMT_BF16, FMT_BF16, 128, BT, false, false);
      const uint32_t id_acc = make_idesc(FMT_BF16, FMT_BF16, 128, D, true, true);
      const uint32_t id_dq = make_idesc(FMT_BF16, FMT_BF16, 128, D, false, true);
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ0 = smem_u32(sQ), aDO = smem_u32(sdO);
      const uint32_t aP = smem_u32(sP), aDS = smem_u32(sdS);
      auto issue_s = [&](int s) {   // S(s) = Q(s)·K^T
        const uint32_t aQ = aQ0 + (s & 1) * Cfg::TILE_BYTES;
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_f16(t_s, make_smem_desc(aQ + off, 0, 1024, 2), make_smem_desc(aK + off, 0, 1024, 2), id_s, kk > 0);
        }
        tc_commit(bars + B_S_FULL);
      };
      auto issue_dp = [&]() {       // dP = dO·V^T
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          mma_f16(t_dp, make_smem_desc(aDO + off, 0, 1024, 2), make_smem_desc(aV + off, 0, 1024, 2), id_s, kk > 0);
        }
        tc_commit(bars + B_DP_FULL);
      };
      bool ok = BWD_WAIT(B_KV_FULL, 0, 3) && BWD_WAIT(B_Q_FULL0, 0, 4);
      if (ok) {
        tc_fence_after();
        issue_s(0);
        ok = BWD_WAIT(B_DO_FULL, 0, 5);
      }
      if (ok) {
        tc_fence_after();
        issue_dp();
        if (n_steps > 1) {
          ok = BWD_WAIT(B_Q_FULL1, 0, 7) && BWD_WAIT(B_S_READ, 0, 8);
          if (ok) { tc_fence_after(); issue_s(1); }
        }
      }
      for (int s = 0; s < n_steps && ok; ++s) {
        const uint32_t aQ = aQ0 + (s & 1) * Cfg::TILE_BYTES;
        BWD_MARK(17)
        ok = BWD_WAIT(B_PDS_READY, s & 1, 9);
        if (!ok) break;
        BWD_MARK(16)
        if (timed) atomicAdd(&phase[23], 1u);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)    // dV += P^T·dO (contraction over the 128 query rows)
          mma_f16(t_dv, make_smem_desc(aP + kk * 2048, 16384, 1024, 2), make_smem_desc(aDO + kk * 2048, 16384, 1024, 2),
                  id_acc, (s > 0 || kk > 0) ? 1u : 0u);
        tc_commit(bars + B_DO_FREE);
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk) {  // dQ(s) = dS·K, contraction over the 128 keys, into dP's columns
          const uint64_t dsa = make_smem_desc(aDS + (kk >> 2) * 16384 + (kk & 3) * 32, 0, 1024, 2);
          mma_f16(t_dp, dsa, make_smem_desc(aK + kk * 2048, 16384, 1024, 2), id_dq, kk > 0);
        }
        tc_commit(bars + B_DQ_FULL);
#pragma unroll
        for (int kk = 0; kk < BT / 16; ++kk)    // dK += dS^T·Q(s)
          mma_f16(t_dk, make_smem_desc(aDS + kk * 2048, 16384, 1024, 2), make_smem_desc(aQ + kk * 2048, 16384, 1024, 2),
                  id_acc, (s > 0 || kk > 0) ? 1u : 0u);
        tc_commit(bars + B_Q_FREE0 + (s & 1));
        if (s + 1 >= n_steps) break;
        BWD_MARK(17)
        ok = BWD_WAIT(B_DQ_DONE, s & 1, 10);
        BWD_MARK(18)
        ok = ok && BWD_WAIT(B_DO_FULL, (s + 1) & 1, 11);
        if (!ok) break;
        BWD_MARK(19)
        tc_fence_after();
        issue_dp();
        if (s + 2 < n_steps) {
          BWD_MARK(17)
          ok = BWD_WAIT(B_Q_FULL0 + (s & 1), ((s + 2) >> 1) & 1, 13);
          BWD_MARK(21)
          ok = ok && BWD_WAIT(B_S_READ, (s + 1) & 1, 14);
          if (!ok) break;
          BWD_MARK(22)
          tc_fence_after();
          issue_s(s + 2);
        }
      }
    }
  } else {
    // -------------------------------------------------------------- softmax / drain warps
    // Two warps share each 32-lane quadrant of tensor memory: warps 0-3 take the first 64
    // columns of S / dP, warps 4-7 the other 64.
    const int r = threadIdx.x & 127, lane = threadIdx.x & 31, half = warp >> 2;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int c_first = half * 64;
    const int base = half * 16384 + r * 128;   // this thread's 128 bytes of the P / dS tiles
    bool ok = true;
    // the step ahead's row statistics, loaded a phase before they are used
    auto row_stats = [&](int s, float& lse2, float& ndlt, int& lo_key, int& hi_key, bool& any_row) {
      const int h = g * hpg + s / per_head;
      const int q = (i_lo + s % per_head) * BT + r;
      const bool row_ok = q < p.T;
      const size_t stat = ((size_t)b * p.H + h) * p.T + (row_ok ? q : 0);
      lse2 = row_ok ? p.lse[stat] * LOG2E_B : 0.f;
      ndlt = row_ok ? -p.delta[stat] * p.scale : 0.f;
      hi_key = p.causal ? q + shift : p.S - 1;
      lo_key = p.window > 0 ? q + shift - p.window + 1 : 0;
      if (p.row_lo != nullptr && row_ok) lo_key = max(lo_key, p.row_lo[(size_t)b * p.T + q]);
      any_row = row_ok && lse2 > -INFINITY;
    };
    float lse2 = 0.f, ndlt = 0.f;
    int lo_key = 0, hi_key = 0;
    bool any_row = false;
    if (n_steps > 0) row_stats(0, lse2, ndlt, lo_key, hi_key, any_row);

    // step s = -1 only prepares step 0 (its P and dS); step n_steps - 1 only drains
    for (int s = -1; s < n_steps && ok; ++s) {
      const bool ahead = s + 1 < n_steps;
      uint32_t pp[32];                          // P(s+1), bf16 pairs, this thread's 64 columns
      const float ndlt_next = ndlt;             // -delta·scale of P(s+1)'s row
      BWD_MARK(13)
      if (ahead) {
        // ---- P(s+1) = exp(S·scale − lse), into registers, while the tensor core runs step s
        const bool full_row = any_row && kv0 + BT - 1 <= hi_key && kv0 >= lo_key && kv0 + BT <= p.S;
        const float nlse2 = -lse2;
        ok = warp_all(BWD_WAIT(B_S_FULL, (s + 1) & 1, 15));
        if (!ok) break;
        BWD_MARK(4)
        tc_fence_after();
        uint32_t cs[2][32];
        tmem_ld_x32(t_s + lane_addr + c_first, cs[0]);
        tmem_ld_x32(t_s + lane_addr + c_first + 32, cs[1]);
#pragma unroll
        for (int ci = 0; ci < 2; ++ci) {
          if (ci == 0) tmem_ld_wait();          // both loads were issued: the second is done as well
#pragma unroll
          for (int i = 0; i < 32; i += 2)
            pp[ci * 16 + (i >> 1)] = pack_bf16(ex2_approx(fmaf(__uint_as_float(cs[ci][i]), p.scale_log2, nlse2)),
                                               ex2_approx(fmaf(__uint_as_float(cs[ci][i + 1]), p.scale_log2, nlse2)));
        }
        tc_fence_before();
        mbar_arrive(bars + B_S_READ);           // S(s+1) is in registers: S(s+2) may overwrite it
        if (!full_row) {
          // rows that the tile's keys only partly see (the diagonal, a window's edge, a document
          // start, the sequence end): the hidden keys' probabilities are cleared afterwards
          const int first = any_row ? max(lo_key - kv0, 0) : BT;          // visible columns: [first, last]
          const int last = min(min(hi_key, p.S - 1) - kv0, BT - 1);
#pragma unroll
          for (int k2 = 0; k2 < 32; ++k2) {
            const int c0 = c_first + 2 * k2;
            const uint32_t keep = (c0 >= first && c0 <= last ? 0x0000ffffu : 0u) |
                                  (c0 + 1 >= first && c0 + 1 <= last ? 0xffff0000u : 0u);
            pp[k2] &= keep;
          }
        }
        if (s + 2 < n_steps) row_stats(s + 2, lse2, ndlt, lo_key, hi_key, any_row);
        BWD_MARK(5)
      }
      if (s >= 0) {
        // ---- dQ(s): tensor memory → registers (dP(s+1) may then be issued) → the P tile and the
        // dS tile, both free once dK(s), the step's last MMA to read them, has run → TMA reduce-adds
        const int h = g * hpg + s / per_head;
        ok = warp_all(BWD_WAIT(B_DQ_FULL, s & 1, 18));
        if (!ok) break;
        BWD_MARK(8)
        tc_fence_after();
        uint32_t v[D / 64][32];
#pragma unroll
        for (int j = 0; j < D / 64; ++j) tmem_ld_x32(t_dp + lane_addr + (half + 2 * j) * 32, v[j]);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(bars + B_DQ_DONE);
        BWD_MARK(9)
        ok = warp_all(BWD_WAIT(B_Q_FREE0 + (s & 1), (s >> 1) & 1, 19));
        if (!ok) break;
        BWD_MARK(10)
        const int row0 = b * p.T + (i_lo + s % per_head) * BT + (warp & 3) * 32;
#pragma unroll
        for (int j = 0; j < D / 64; ++j) {
          uint8_t* tile = j == 0 ? sP : sdS;
#pragma unroll
          for (int sl = 0; sl < 8; ++sl)
            *reinterpret_cast<uint4*>(tile + base + ((sl ^ (r & 7)) << 4)) =
                make_uint4(v[j][4 * sl], v[j][4 * sl + 1], v[j][4 * sl + 2], v[j][4 * sl + 3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
#pragma unroll
          for (int j = 0; j < D / 64; ++j)
            tma_reduce_add_2d(&p.tmap_dq, (j == 0 ? sP : sdS) + half * 16384 + (warp & 3) * 4096,
                              h * D + (half + 2 * j) * 32, row0);
          tma_store_commit();
        }
        BWD_MARK(11)
      }
      if (ahead) {
        // ---- dS(s+1) = P∘(dP·scale − delta·scale), then both tiles of step s+1 are stored
        ok = warp_all(BWD_WAIT(B_DP_FULL, (s + 1) & 1, 17));
        if (!ok) break;
        BWD_MARK(0)
        tc_fence_after();
        uint32_t ds[32];
        uint32_t cd[2][32];
        tmem_ld_x32(t_dp + lane_addr + c_first, cd[0]);
        tmem_ld_x32(t_dp + lane_addr + c_first + 32, cd[1]);
        tmem_ld_wait();
#pragma unroll
        for (int ci = 0; ci < 2; ++ci) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float2 pv = unpack_bf16(pp[ci * 16 + (i >> 1)]);
            ds[ci * 16 + (i >> 1)] = pack_bf16(pv.x * fmaf(__uint_as_float(cd[ci][i]), p.scale, ndlt_next),
                                               pv.y * fmaf(__uint_as_float(cd[ci][i + 1]), p.scale, ndlt_next));
          }
        }
        tc_fence_before();
        BWD_MARK(1)
        // both halves of dQ(s) were staged in this warp's rows of the two tiles
        if (lane == 0) tma_store_wait_read();
        __syncwarp();
        BWD_MARK(2)
#pragma unroll
        for (int sl = 0; sl < 8; ++sl) {
          *reinterpret_cast<uint4*>(sP + base + ((sl ^ (r & 7)) << 4)) =
              make_uint4(pp[4 * sl], pp[4 * sl + 1], pp[4 * sl + 2], pp[4 * sl + 3]);
          *reinterpret_cast<uint4*>(sdS + base + ((sl ^ (r & 7)) << 4)) =
              make_uint4(ds[4 * sl], ds[4 * sl + 1], ds[4 * sl + 2], ds[4 * sl + 3]);
        }
        fence_proxy_async_smem();
        mbar_arrive(bars + B_PDS_READY);
        BWD_MARK(3)
      }
    }
    if (lane == 0) tma_store_wait_all();
    __syncwarp();
    // the last step's dK (and with it every MMA of the walk) is complete
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
  if (p.phase_cycles != nullptr && (blockIdx.x | blockIdx.y | blockIdx.z) == 0 && threadIdx.x < 32)
    atomicAdd(&p.phase_cycles[threadIdx.x], phase[threadIdx.x]);
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
  p.status = a.status; p.phase_cycles = a.phase_cycles;
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
