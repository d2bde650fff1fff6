// Chunkwise linear recurrence (delta rule and decayed linear attention) for sm_100a: the part of
// the scan that runs from chunk to chunk, on tcgen05 tensor cores with the state in tensor memory.
//
// A recurrence  S_t = diag(w_t) S_{t-1} + b_t (a_t^T S_{t-1}) + k_t v_t^T,  o_t = q_t^T S_t  is cut
// into chunks of 64 positions. What a chunk needs from inside itself (the decayed pair matrices,
// the inverse of the unit-triangular system of the rank-one term) is independent of every other
// chunk and is formed beforehand for all chunks at once. What is left is serial in the chunks:
//
//   X  = P S + W V                      the rank-one term's reads of the state      [64, dv]
//   O  = Qd S + Mqk V + Mqb X           the chunk's outputs                         [64, dv]
//   S' = diag(lam) S + Kd^T V + Bd^T X  the state after the chunk                   [dk, dv]
//
// One CTA walks the chunks of one (row, head). Per chunk, four chains of 128-row MMAs:
//   Y  = [P; Qd] S        (A from shared memory, S as a bf16 copy in shared memory)
//   Y += [W; Mqk] V       rows 0-63 of Y are X, rows 64-127 are O without its X term
//   Y += [0; Mqb] X       X written to shared memory by the warps that read it from Y
//   S += [Kd; Bd]^T [V; X]   accumulated in tensor memory, where diag(lam) S was left
// Between chunks the four warps read S out of tensor memory, leave a bf16 copy for the next
// chunk's first chain (and, when asked, in global memory for the backward), scale it by the next
// chunk's decay and write it back. The state never leaves the SM in fp32 until the last chunk.
//
// The backward of the serial part has the same shape with other operands and the chunks walked
// from last to first (dX = Bd dS' + Mqb^T dO;  dS = diag(lam) dS' + [Qd; P]^T [dO; dX]), so this
// kernel serves both directions: `reverse`, and `has_out = false` skip the output chain.
//
// Reference counterparts: architecture/recurrent/chunkwise.py:40-441 (XLA einsums),
// affine_scan.py:120-149 (the scan across chunks), fused_delta.py:229-335 (cuDNN's fused kernels).
#include "common.cuh"
#include "gemm_sm100.h"
#include "scan_sm100.h"

namespace bux {

constexpr int KID_SCAN = 6;
constexpr int SCAN_THREADS = 192;  // 4 warps on the tensor-memory lanes, TMA warp, MMA warp
constexpr int CH = 64;             // positions per chunk
constexpr int DK = 128, DV = 128;  // padded head dims

struct ScanParams {
  alignas(64) CUtensorMap tm_a1;    // [BH*n*128, DK]   rows 0-63 P (bwd: Bd), 64-127 Qd (bwd: 0)
  alignas(64) CUtensorMap tm_aux1;  // [BH*n*128, 64]   rows 0-63 W (bwd: Mqb^T), 64-127 Mqk (bwd: 0)
  alignas(64) CUtensorMap tm_aux3;  // [BH*n*64, 64]    Mqb
  alignas(64) CUtensorMap tm_a4;    // [BH*n*128, DK]   rows 0-63 Kd (bwd: Qd), 64-127 Bd (bwd: P)
  alignas(64) CUtensorMap tm_v;     // [BH*n*64, DV]    V (bwd: dO)
  const float* lam;                 // [BH*n, DK] decay of the state over each chunk
  const float* s0;                  // [BH, DK, DV] or null
  __nv_bfloat16* out;               // [BH*n*64, DV] or null
  __nv_bfloat16* x_out;             // [BH*n*64, DV] or null
  __nv_bfloat16* states;            // [BH*n, DK, DV] the state each chunk starts from, or null
  float* s_last;                    // [BH, DK, DV]
  Status* status;
  int n_chunks, reverse, has_out;
};

enum ScanBar { SB_L1_FULL = 0, SB_L2_FULL, SB_Y1_FULL, SB_X_READY, SB_Y3_FULL, SB_Y_FREE, SB_S_FULL, SB_S_READY, SB_COUNT };

constexpr int SCAN_SMEM = 32768 /*A1*/ + 16384 /*aux1*/ + 16384 /*aux3*/ + 32768 /*A4*/ + 32768 /*VX*/ +
                          32768 /*S*/ + 1024 + 256;

__global__ void __launch_bounds__(SCAN_THREADS, 1) chunk_scan_kernel(const __grid_constant__ ScanParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sA1 = smem;
  uint8_t* sAux1 = sA1 + 32768;
  uint8_t* sAux3 = sAux1 + 16384;
  uint8_t* sA4 = sAux3 + 16384;
  uint8_t* sVX = sA4 + 32768;
  uint8_t* sS = sVX + 32768;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sS + 32768);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + SB_COUNT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int bh = blockIdx.x, n = p.n_chunks;
  Status* st = p.status;
  auto chunk_at = [&](int i) { return p.reverse ? n - 1 - i : i; };   // i-th chunk of the walk

  if (threadIdx.x == 0) {
    mbar_init(bars + SB_L1_FULL, 1); mbar_init(bars + SB_L2_FULL, 1);
    mbar_init(bars + SB_Y1_FULL, 1); mbar_init(bars + SB_X_READY, 64);
    mbar_init(bars + SB_Y3_FULL, 1); mbar_init(bars + SB_Y_FREE, 64);
    mbar_init(bars + SB_S_FULL, 1); mbar_init(bars + SB_S_READY, 128);
    *abort_flag = 0;
    mbar_fence_init();
  }
  // rows 0-63 of the [0; Mqb] operand stay zero
  for (int i = threadIdx.x; i < 8192 / 16; i += SCAN_THREADS) reinterpret_cast<uint4*>(sAux3)[i] = make_uint4(0, 0, 0, 0);
  fence_proxy_async_smem();
  if (warp == 5) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t t_y = tmem_base, t_s = tmem_base + 128;
#define SCAN_WAIT(slot, parity, site) mbar_wait(bars + (slot), (parity), abort_flag, st, KID_SCAN, (site))

  if (warp == 4) {
    // -------------------------------------------------------------- TMA producer
    if (elect_one()) {
      for (int i = 0; i < n; ++i) {
        const int row128 = (bh * n + chunk_at(i)) * 128, row64 = (bh * n + chunk_at(i)) * 64;
        if (i > 0 && !SCAN_WAIT(SB_Y1_FULL, (i - 1) & 1, 1)) break;     // the first two chains have read A1 / aux1
        mbar_expect_tx(bars + SB_L1_FULL, 32768 + 16384);
        tma_load_2d(sA1, &p.tm_a1, 0, row128, bars + SB_L1_FULL);
        tma_load_2d(sA1 + 16384, &p.tm_a1, 64, row128, bars + SB_L1_FULL);
        tma_load_2d(sAux1, &p.tm_aux1, 0, row128, bars + SB_L1_FULL);
        if (i > 0 && !SCAN_WAIT(SB_S_FULL, (i - 1) & 1, 2)) break;      // the last chain has read A4, V, X, Mqb
        mbar_expect_tx(bars + SB_L2_FULL, (p.has_out ? 8192 : 0) + 16384 + 32768);
        if (p.has_out) tma_load_2d(sAux3 + 8192, &p.tm_aux3, 0, row64, bars + SB_L2_FULL);
        tma_load_2d(sVX, &p.tm_v, 0, row64, bars + SB_L2_FULL);
        tma_load_2d(sVX + 16384, &p.tm_v, 64, row64, bars + SB_L2_FULL);
        tma_load_2d(sA4, &p.tm_a4, 0, row128, bars + SB_L2_FULL);
        tma_load_2d(sA4 + 16384, &p.tm_a4, 64, row128, bars + SB_L2_FULL);
      }
    }
  } else if (warp == 5) {
    // -------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t id_kn = make_idesc(FMT_BF16, FMT_BF16, 128, DV, false, true);   // A K-major, B rows along K
      const uint32_t id_mn = make_idesc(FMT_BF16, FMT_BF16, 128, DV, true, true);    // A rows along K as well
      const uint32_t aA1 = smem_u32(sA1), aAux1 = smem_u32(sAux1), aAux3 = smem_u32(sAux3), aA4 = smem_u32(sA4);
      const uint32_t aVX = smem_u32(sVX), aS = smem_u32(sS);
      bool ok = true;
      for (int i = 0; i < n && ok; ++i) {
        ok = SCAN_WAIT(SB_L1_FULL, i & 1, 3) && SCAN_WAIT(SB_S_READY, i & 1, 4);
        if (ok && i > 0 && p.has_out) ok = SCAN_WAIT(SB_Y_FREE, (i - 1) & 1, 5);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < DK / 16; ++kk)   // Y = [P; Qd] S
          mma_f16(t_y, make_smem_desc(aA1 + (kk >> 2) * 16384 + (kk & 3) * 32, 0, 1024, 2),
                  make_smem_desc(aS + kk * 2048, 16384, 1024, 2), id_kn, kk > 0);
        ok = SCAN_WAIT(SB_L2_FULL, i & 1, 6);
        if (!ok) break;
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < CH / 16; ++kk)   // Y += [W; Mqk] V
          mma_f16(t_y, make_smem_desc(aAux1 + kk * 32, 0, 1024, 2), make_smem_desc(aVX + kk * 2048, 16384, 1024, 2),
                  id_kn, 1u);
        tc_commit(bars + SB_Y1_FULL);
        ok = SCAN_WAIT(SB_X_READY, i & 1, 7);
        if (!ok) break;
        tc_fence_after();
        if (p.has_out) {
#pragma unroll
          for (int kk = 0; kk < CH / 16; ++kk)  // Y += [0; Mqb] X
            mma_f16(t_y, make_smem_desc(aAux3 + kk * 32, 0, 1024, 2),
                    make_smem_desc(aVX + (4 + kk) * 2048, 16384, 1024, 2), id_kn, 1u);
          tc_commit(bars + SB_Y3_FULL);
        }
#pragma unroll
        for (int kk = 0; kk < 128 / 16; ++kk)   // S += [Kd; Bd]^T [V; X]
          mma_f16(t_s, make_smem_desc(aA4 + kk * 2048, 16384, 1024, 2), make_smem_desc(aVX + kk * 2048, 16384, 1024, 2),
                  id_mn, 1u);
        tc_commit(bars + SB_S_FULL);
      }
    }
  } else {
    // -------------------------------------------------------------- the four warps on the lanes
    const int row = threadIdx.x;                       // tensor-memory lane = row of Y and of S
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    bool ok = true;
    // a 32-column piece of this thread's row of a [128 x 128] bf16 tile (two 64-column halves)
    auto store_tile = [&](uint8_t* tile, int r, int c32, const uint32_t (&v)[32]) {
      uint8_t* line = tile + (c32 >> 1) * 16384 + r * 128;
#pragma unroll
      for (int sl = 0; sl < 4; ++sl) {
        const int slot = ((c32 & 1) << 2) + sl;
        *reinterpret_cast<uint4*>(line + ((slot ^ (r & 7)) << 4)) =
            make_uint4(pack_bf16(__uint_as_float(v[8 * sl]), __uint_as_float(v[8 * sl + 1])),
                       pack_bf16(__uint_as_float(v[8 * sl + 2]), __uint_as_float(v[8 * sl + 3])),
                       pack_bf16(__uint_as_float(v[8 * sl + 4]), __uint_as_float(v[8 * sl + 5])),
                       pack_bf16(__uint_as_float(v[8 * sl + 6]), __uint_as_float(v[8 * sl + 7])));
      }
    };
    auto store_global = [&](__nv_bfloat16* dst, const uint32_t (&v)[32]) {   // 32 values as bf16, 64 bytes
#pragma unroll
      for (int sl = 0; sl < 4; ++sl)
        reinterpret_cast<uint4*>(dst)[sl] =
            make_uint4(pack_bf16(__uint_as_float(v[8 * sl]), __uint_as_float(v[8 * sl + 1])),
                       pack_bf16(__uint_as_float(v[8 * sl + 2]), __uint_as_float(v[8 * sl + 3])),
                       pack_bf16(__uint_as_float(v[8 * sl + 4]), __uint_as_float(v[8 * sl + 5])),
                       pack_bf16(__uint_as_float(v[8 * sl + 6]), __uint_as_float(v[8 * sl + 7])));
    };
    // the state this walk starts from: a bf16 copy for the first chunk's first chain, the state
    // scaled by the first chunk's decay into tensor memory
    {
      const float l0 = p.lam[(size_t)(bh * n + chunk_at(0)) * DK + row];
#pragma unroll 1
      for (int c32 = 0; c32 < DV / 32; ++c32) {
        uint32_t v[32];
#pragma unroll
        for (int i = 0; i < 32; ++i)
          v[i] = p.s0 ? __float_as_uint(p.s0[((size_t)bh * DK + row) * DV + c32 * 32 + i]) : 0u;
        store_tile(sS, row, c32, v);
        if (p.states) store_global(p.states + ((size_t)(bh * n + chunk_at(0)) * DK + row) * DV + c32 * 32, v);
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * l0);
        tmem_st_x32(t_s + lane_addr + c32 * 32, v);
      }
      tmem_st_wait();
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(bars + SB_S_READY);
    }
    for (int i = 0; i < n && ok; ++i) {
      const int ci = chunk_at(i);
      if (warp < 2) {
        // ---- X = rows 0-63 of Y: into the lower half of the [V; X] tile (and global memory)
        ok = warp_all(SCAN_WAIT(SB_Y1_FULL, i & 1, 8));
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c32 = 0; c32 < DV / 32; ++c32) {
          uint32_t v[32];
          tmem_ld_x32(t_y + lane_addr + c32 * 32, v);
          tmem_ld_wait();
          store_tile(sVX, 64 + row, c32, v);
          if (p.x_out) store_global(p.x_out + ((size_t)(bh * n + ci) * CH + row) * DV + c32 * 32, v);
        }
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(bars + SB_X_READY);
      } else if (p.has_out) {
        // ---- O = rows 64-127 of Y after the X term
        ok = warp_all(SCAN_WAIT(SB_Y3_FULL, i & 1, 9));
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c32 = 0; c32 < DV / 32; ++c32) {
          uint32_t v[32];
          tmem_ld_x32(t_y + lane_addr + c32 * 32, v);
          tmem_ld_wait();
          store_global(p.out + ((size_t)(bh * n + ci) * CH + (row - 64)) * DV + c32 * 32, v);
        }
        tc_fence_before();
        mbar_arrive(bars + SB_Y_FREE);
      }
      // ---- the state after the chunk: bf16 copy for the next chunk, decay of the next chunk
      ok = warp_all(SCAN_WAIT(SB_S_FULL, i & 1, 10));
      if (!ok) break;
      tc_fence_after();
      const bool last = i + 1 == n;
      const int cn = last ? 0 : chunk_at(i + 1);
      const float ln = last ? 1.f : p.lam[(size_t)(bh * n + cn) * DK + row];
#pragma unroll 1
      for (int c32 = 0; c32 < DV / 32; ++c32) {
        uint32_t v[32];
        tmem_ld_x32(t_s + lane_addr + c32 * 32, v);
        tmem_ld_wait();
        if (last) {
#pragma unroll
          for (int q = 0; q < 8; ++q)
            reinterpret_cast<uint4*>(p.s_last + ((size_t)bh * DK + row) * DV + c32 * 32)[q] =
                make_uint4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
        } else {
          store_tile(sS, row, c32, v);
          if (p.states) store_global(p.states + ((size_t)(bh * n + cn) * DK + row) * DV + c32 * 32, v);
#pragma unroll
          for (int q = 0; q < 32; ++q) v[q] = __float_as_uint(__uint_as_float(v[q]) * ln);
          tmem_st_x32(t_s + lane_addr + c32 * 32, v);
        }
      }
      if (!last) {
        tmem_st_wait();
        tc_fence_before();
        fence_proxy_async_smem();
        mbar_arrive(bars + SB_S_READY);
      }
    }
    (void)lane;
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

const char* chunk_scan_launch(const ScanArgs& a, cudaStream_t stream) {
  if (a.dk != DK || a.dv != DV) return "chunk_scan: head dims must be padded to 128";
  if (a.n_chunks < 1 || a.bh < 1) return "chunk_scan: nothing to do";
  ScanParams p;
  const char* err;
  const uint64_t r128 = (uint64_t)a.bh * a.n_chunks * 128, r64 = (uint64_t)a.bh * a.n_chunks * 64;
  if ((err = make_tmap_2d(&p.tm_a1, a.a1, 2, r128, DK, DK * 2, 64, 128))) return err;
  if ((err = make_tmap_2d(&p.tm_aux1, a.aux1, 2, r128, 64, 64 * 2, 64, 128))) return err;
  if ((err = make_tmap_2d(&p.tm_aux3, a.aux3 ? a.aux3 : a.aux1, 2, a.aux3 ? r64 : r128, 64, 64 * 2, 64, 64))) return err;
  if ((err = make_tmap_2d(&p.tm_a4, a.a4, 2, r128, DK, DK * 2, 64, 128))) return err;
  if ((err = make_tmap_2d(&p.tm_v, a.v, 2, r64, DV, DV * 2, 64, 64))) return err;
  p.lam = a.lam; p.s0 = a.s0; p.out = reinterpret_cast<__nv_bfloat16*>(a.out);
  p.x_out = reinterpret_cast<__nv_bfloat16*>(a.x_out); p.states = reinterpret_cast<__nv_bfloat16*>(a.states);
  p.s_last = a.s_last; p.status = a.status;
  p.n_chunks = a.n_chunks; p.reverse = a.reverse ? 1 : 0; p.has_out = (a.out != nullptr && a.aux3 != nullptr) ? 1 : 0;
  static bool configured[64] = {};
  if (!allow_dynamic_smem(chunk_scan_kernel, SCAN_SMEM, configured))
    return "cudaFuncSetAttribute(max dynamic shared memory) failed";
  chunk_scan_kernel<<<a.bh, SCAN_THREADS, SCAN_SMEM, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? nullptr : "chunk_scan launch failed";
}

}  // namespace bux
