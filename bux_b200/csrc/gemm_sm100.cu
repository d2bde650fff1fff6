// Persistent warp-specialised tcgen05 GEMM for sm_100a: bf16 and block-scaled MXFP8,
// dense, grouped-by-rows (MoE experts, ragged M) and grouped-by-contraction (expert
// weight gradients, ragged K).
//
//   C[M,N] (+)= A · B^T           A: [M,K]  B: [N,K]   (both "K-major"), or either operand
//                                 stored transposed ("MN-major": A as [K,M], B as [K,N]).
//
// Roles per CTA (192 threads, one CTA per SM):
//   warp 0      one elected lane issues TMA loads (non-multicast) into a ring of stages
//   warp 1      one elected lane issues tcgen05.mma into a TMEM accumulator and commits
//               stage-free / accumulator-full mbarriers; allocates and frees TMEM
//   warps 2..5  epilogue: tcgen05.ld the accumulator (each warp its 32-lane quadrant),
//               convert, store (bf16 / fp32 / fp32 accumulate), masked at ragged edges
// The accumulator is double-buffered in TMEM so tile i's epilogue overlaps tile i+1's
// main loop. MXFP8 scale factors travel global -> smem by bulk copy (they are stored
// pre-tiled, 512 bytes per 128 rows x 128 K) and smem -> TMEM by tcgen05.cp.
//
// Counterparts in the reference: cuBLAS/cuDNN GEMMs behind XLA dots
// (architecture/precision/blockscaled.py:204) and the Mosaic-GPU grouped kernel
// (architecture/experts/grouped_mxfp8.py:416-740). Unlike the latter, no load here is
// a cluster-multicast load.
#include <cstdio>

#include "common.cuh"
#include "gemm_sm100.h"

namespace bux {

constexpr int KID_GEMM = 1;
constexpr int BM = 128;

template <int KIND, int BN, int EW = 4>
struct GemmCfg {
  // bytes of K per stage row: 128 for both kinds (64 bf16 or 128 fp8)
  static constexpr int BK_ELEMS = KIND == KIND_BF16 ? 64 : 128;
  static constexpr int ELEM = KIND == KIND_BF16 ? 2 : 1;
  static constexpr int A_BYTES = BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int SF_BYTES = KIND == KIND_MXFP8 ? 512 * (1 + BN / 128) : 0;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SF_BYTES;
  // epilogue staging: per warp 32 rows x 64 bf16 columns (4 KB), one or two slabs per warp.
  // The 256-wide MXFP8 tile has room for one accumulator only (two would leave no TMEM columns
  // for the scales), so its epilogue is not hidden behind the next tile's MMAs. Eight epilogue
  // warps (EW = 8: two per TMEM lane quadrant, half the columns each) drain it in half the
  // time, but their slabs cost a pipeline stage: measured 4 % faster on the grouped expert
  // GEMMs and 5 % slower on the dense ones, so the launcher takes eight for grouped rows only.
  static constexpr bool ONE_ACC = KIND == KIND_MXFP8 && BN == 256;
  static constexpr int EPI_WARPS = EW;
  static constexpr int THREADS = 64 + 32 * EPI_WARPS;
  static constexpr int EPI_SLABS = ONE_ACC ? 1 : 2;
  static constexpr int EPI_BYTES = EPI_SLABS * EPI_WARPS * 4096;
  static constexpr int BUDGET = 227 * 1024 - 1024 - 256 - 1024 - EPI_BYTES;
  static constexpr int STAGES = BUDGET / STAGE_BYTES > 8 ? 8 : BUDGET / STAGE_BYTES;
  static constexpr int ACC_STAGES = (2 * BN + (KIND == KIND_MXFP8 ? STAGES * 4 * (1 + BN / 128) : 0)) <= 512 ? 2 : 1;
  static constexpr int ACC_COLS = ACC_STAGES * BN;
  static constexpr int SF_COLS_PER_STAGE = KIND == KIND_MXFP8 ? 4 * (1 + BN / 128) : 0;
  static constexpr int TMEM_COLS = 512;
  static constexpr int UMMA_K = KIND == KIND_BF16 ? 16 : 32;
  static constexpr int EPI_OFFSET = (STAGES * STAGE_BYTES + 1023) / 1024 * 1024;
  static constexpr int SMEM_BYTES = EPI_OFFSET + EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

struct TileCoord {
  int group;    // expert index (0 when dense)
  int m0;       // first row of A / C (global row in the sorted layout for MODE_GROUPED_ROWS)
  int m_end;    // one past the last valid row
  int n0;
  int k0, k1;   // contraction range in elements
  bool valid;
};

// Deterministic tile walk shared by all roles. Dense tiles are rasterised in
// super-rows of 16 m-tiles so one wave's A and B tiles stay L2-resident.
struct TileWalk {
  const GemmParams& p;
  int n_tiles, bn;
  int t;            // linear tile index of this CTA
  int g;            // group cursor (grouped modes)
  int tiles_before; // tiles of groups < g
  __device__ TileWalk(const GemmParams& p_, int bn_) : p(p_), n_tiles((p_.N + bn_ - 1) / bn_), bn(bn_), t(blockIdx.x), g(0), tiles_before(0) {}

  __device__ TileCoord next() {
    TileCoord c;
    c.valid = false;
    if (p.mode == MODE_DENSE) {
      int m_tiles = (p.M + BM - 1) / BM;
      int total = m_tiles * n_tiles;
      if (t >= total) return c;
      constexpr int GM = 16;
      int per_super = GM * n_tiles;
      int sup = t / per_super, local = t % per_super;
      int rows_here = min(GM, m_tiles - sup * GM);
      int mt = sup * GM + local % rows_here;
      int nt = local / rows_here;
      if (p.m_rotate) mt = (mt + p.m_rotate) % m_tiles;
      c.group = 0; c.m0 = mt * BM; c.m_end = p.M; c.n0 = nt * bn; c.k0 = 0; c.k1 = p.K;
      c.valid = true;
    } else if (p.mode == MODE_GROUPED_ROWS) {
      while (g < p.groups) {
        int r0 = p.group_offsets[g], r1 = p.group_offsets[g + 1];
        int mt_g = (r1 - r0 + BM - 1) / BM;
        int here = mt_g * n_tiles;
        if (t < tiles_before + here) {
          int local = t - tiles_before;
          c.group = g; c.m0 = r0 + (local % mt_g) * BM; c.m_end = r1; c.n0 = (local / mt_g) * bn;
          c.k0 = 0; c.k1 = p.K; c.valid = true;
          break;
        }
        tiles_before += here;
        ++g;
      }
    } else {  // MODE_GROUPED_K: every group has the same M x N output, its own K range
      int m_tiles = (p.M + BM - 1) / BM;
      int per_group = m_tiles * n_tiles;
      if (t >= per_group * p.groups) return c;
      int gi = t / per_group, local = t % per_group;
      c.group = gi; c.m0 = (local % m_tiles) * BM; c.m_end = p.M; c.n0 = (local / m_tiles) * bn;
      c.k0 = p.group_offsets[gi]; c.k1 = p.group_offsets[gi + 1]; c.valid = true;
    }
    t += gridDim.x;
    return c;
  }
};

template <int KIND, int BN, bool A_MN, bool B_MN, int EW = 4>
__global__ void __launch_bounds__((GemmCfg<KIND, BN, EW>::THREADS), 1)
gemm_sm100_kernel(const __grid_constant__ GemmParams p) {
  using Cfg = GemmCfg<KIND, BN, EW>;
  constexpr int STAGES = Cfg::STAGES;
  constexpr int ACC_STAGES = Cfg::ACC_STAGES;
  extern __shared__ uint8_t smem_raw[];
  // 1024-byte alignment: the 128B-swizzle atom is 8 rows x 128 bytes.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // the epilogue slabs swizzle by address bits 7-9: they start on a 1024-byte boundary
  uint8_t* epi_smem = smem + Cfg::EPI_OFFSET;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi_smem + Cfg::EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + STAGES;
  uint64_t* acc_full = bars + 2 * STAGES;
  uint64_t* acc_empty = acc_full + ACC_STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  Status* st = p.status;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < ACC_STAGES; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], Cfg::EPI_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, Cfg::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      tma_prefetch_desc(&p.tmap_a);
      tma_prefetch_desc(&p.tmap_b);
      TileWalk walk(p, BN);
      int stage = 0; uint32_t phase = 0;
      bool ok = true;
      uint32_t seen = 0;  // senders whose flag this CTA has seen (wait_rows mode)
      auto wait_sender = [&](int r) -> bool {
        if (r >= p.wait_world) r = p.wait_world - 1;
        if (seen >> r & 1u) return true;
        const uint64_t t0 = global_ns();
        int v;
        do {
          asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.wait_flags + r) : "memory");
          if (v >= p.wait_epoch) break;
          if (global_ns() - t0 > p.wait_limit_ns) { *abort_flag = 1; report_failure(st, KID_GEMM, 6); return false; }
          __nanosleep(100);
        } while (true);
        asm volatile("fence.proxy.async.global;" ::: "memory");
        seen |= 1u << r;
        return true;
      };
      if (p.wait_flags != nullptr && p.wait_rows == 0) {
        // operand A is being written by peer GPUs: wait for every sender's flag
        const uint64_t t0 = global_ns();
        for (int r = 0; r < p.wait_world && ok; ++r) {
          int v;
          do {
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.wait_flags + r) : "memory");
            if (v >= p.wait_epoch) break;
            if (global_ns() - t0 > p.wait_limit_ns) { ok = false; *abort_flag = 1; report_failure(st, KID_GEMM, 5); break; }
            __nanosleep(100);
          } while (true);
        }
        // order the TMA (async proxy) reads after the flags were seen
        asm volatile("fence.proxy.async.global;" ::: "memory");
      }
      for (TileCoord c = walk.next(); c.valid && ok; c = walk.next()) {
        const int b_row0 = (p.mode == MODE_GROUPED_ROWS ? c.group * p.N : 0) + c.n0;
        // MN-major B of a grouped-rows GEMM is stored [groups * K, N]
        const int b_k_off = (B_MN && p.mode == MODE_GROUPED_ROWS) ? c.group * p.K : 0;
        if (p.wait_flags != nullptr && p.wait_rows > 0 && p.wait_on_n) {
          // operand B's rows (output columns) arrive sender by sender: a weight gathered from its shards
          if (!wait_sender(c.n0 / p.wait_rows) || !wait_sender((min(c.n0 + BN, p.N) - 1) / p.wait_rows)) { ok = false; break; }
        } else if (p.wait_flags != nullptr && p.wait_rows > 0 && !p.wait_on_k) {
          // a tile may straddle two senders' row blocks
          if (!wait_sender(c.m0 / p.wait_rows) || !wait_sender((min(c.m0 + BM, p.M) - 1) / p.wait_rows)) { ok = false; break; }
        }
        for (int k = c.k0; k < c.k1; k += Cfg::BK_ELEMS) {
          if (p.wait_flags != nullptr && p.wait_rows > 0 && p.wait_on_k && !p.wait_on_n) {
            if (!wait_sender(k / p.wait_rows) || !wait_sender((min(k + Cfg::BK_ELEMS, c.k1) - 1) / p.wait_rows)) { ok = false; break; }
          }
          if (!mbar_wait(&empty[stage], phase ^ 1, abort_flag, st, KID_GEMM, 1)) { ok = false; break; }
          uint8_t* sa = smem + stage * Cfg::STAGE_BYTES;
          uint8_t* sb = sa + Cfg::A_BYTES;
          mbar_expect_tx(&full[stage], Cfg::A_BYTES + Cfg::B_BYTES + Cfg::SF_BYTES);
          if (A_MN) {
            // A stored [K, M]: boxes of 64 m-elements x BK k-rows
            for (int j = 0; j < BM / 64; ++j)
              tma_load_2d(sa + j * (Cfg::BK_ELEMS * 128), &p.tmap_a, c.m0 + j * 64, k, &full[stage]);
          } else {
            tma_load_2d(sa, &p.tmap_a, k, c.m0, &full[stage]);
          }
          if (B_MN) {
            for (int j = 0; j < BN / 64; ++j)
              tma_load_2d(sb + j * (Cfg::BK_ELEMS * 128), &p.tmap_b, c.n0 + j * 64, b_k_off + k, &full[stage]);
          } else {
            tma_load_2d(sb, &p.tmap_b, k, b_row0, &full[stage]);
          }
          if (KIND == KIND_MXFP8) {
            uint8_t* ssf = sb + Cfg::B_BYTES;
            const int kb = k / 128;
            const int kblocks = p.k_total / 128;
            bulk_load(ssf, p.sfa + ((size_t)(c.m0 / 128) * kblocks + kb) * 512, 512, &full[stage]);
            for (int j = 0; j < BN / 128; ++j)
              bulk_load(ssf + 512 * (1 + j), p.sfb + ((size_t)(b_row0 / 128 + j) * kblocks + kb) * 512, 512, &full[stage]);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      TileWalk walk(p, BN);
      int stage = 0; uint32_t phase = 0;
      int acc = 0; uint32_t acc_phase = 0;
      bool ok = true;
      for (TileCoord c = walk.next(); c.valid && ok; c = walk.next()) {
        if (!mbar_wait(&acc_empty[acc], acc_phase ^ 1, abort_flag, st, KID_GEMM, 2)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        uint32_t accumulate = 0;
        if (c.k0 >= c.k1) {
          // an empty contraction range (an expert with no tokens): nothing was loaded
        }
        for (int k = c.k0; k < c.k1; k += Cfg::BK_ELEMS) {
          if (!mbar_wait(&full[stage], phase, abort_flag, st, KID_GEMM, 3)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + stage * Cfg::STAGE_BYTES);
          const uint32_t sb = sa + Cfg::A_BYTES;
          uint32_t sf_tmem = 0;
          if (KIND == KIND_MXFP8) {
            sf_tmem = tmem_base + Cfg::ACC_COLS + stage * Cfg::SF_COLS_PER_STAGE;
            const uint32_t ssf = sb + Cfg::B_BYTES;
#pragma unroll
            for (int j = 0; j < 1 + BN / 128; ++j)
              tmem_cp_sf(sf_tmem + 4 * j, make_smem_desc(ssf + 512 * j, 0, 128, 0));
          }
#pragma unroll
          for (int kk = 0; kk < Cfg::BK_ELEMS / Cfg::UMMA_K; ++kk) {
            uint64_t ad, bd;
            if (A_MN) ad = make_smem_desc(sa + kk * 2048, Cfg::BK_ELEMS * 128, 1024, 2);
            else      ad = make_smem_desc(sa + kk * 32, 0, 1024, 2);
            if (B_MN) bd = make_smem_desc(sb + kk * 2048, Cfg::BK_ELEMS * 128, 1024, 2);
            else      bd = make_smem_desc(sb + kk * 32, 0, 1024, 2);
            if (KIND == KIND_BF16) {
              mma_f16(d_tmem, ad, bd, make_idesc(FMT_BF16, FMT_BF16, BM, BN, A_MN, B_MN), accumulate);
            } else {
              mma_mxf8(d_tmem, ad, bd, make_idesc_mx(FMT_E4M3, FMT_E4M3, BM, BN, kk, kk),
                       sf_tmem, sf_tmem + 4, accumulate);
            }
            accumulate = 1;
          }
          tc_commit(&empty[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1; }
        }
        if (!ok) break;
        tc_commit(&acc_full[acc]);
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int quad = warp & 3;  // TMEM lane quadrant this warp may read
    // with eight epilogue warps, warps 2-5 take the tile's first half of the columns, 6-9 the second
    constexpr int EPI_COLS = BN * 4 / Cfg::EPI_WARPS;
    const int col_begin = ((warp - 2) >> 2) * EPI_COLS;
    TileWalk walk(p, BN);
    int acc = 0; uint32_t acc_phase = 0;
    int epi_round = 0;
    bool ok = true;
    for (TileCoord c = walk.next(); c.valid && ok; c = walk.next()) {
      if (!warp_all(mbar_wait(&acc_full[acc], acc_phase, abort_flag, st, KID_GEMM, 4))) { ok = false; break; }
      tc_fence_after();
      const int row = c.m0 + quad * 32 + lane;
      const bool row_ok = row < c.m_end;
      const bool empty_k = c.k0 >= c.k1;
      size_t out_row = (size_t)row;
      if (p.mode == MODE_GROUPED_K) out_row += (size_t)c.group * p.M;
      const uint32_t t_addr = tmem_base + acc * BN + ((uint32_t)(quad * 32) << 16);
      // full bf16 tiles leave through shared memory and TMA stores: whole 128-byte lines,
      // asynchronous, and the accumulator is released as soon as it has been read
      const bool by_tma = p.tma_store && (p.mode != MODE_GROUPED_ROWS || c.m_end - c.m0 >= BM);
      const bool out_bf16 = p.out_kind == OUT_BF16 || p.out_kind == OUT_BF16_ACC;
      const bool out_adds = p.out_kind == OUT_F32_ACC || p.out_kind == OUT_BF16_ACC;
      if (by_tma) {
        uint8_t* mine = epi_smem + (warp - 2) * 4096;
        const int out_row0 = (p.mode == MODE_GROUPED_K ? c.group * p.M : 0) + c.m0 + quad * 32;
        // a slab is 32 rows x 128 bytes: 64 bf16 columns, or 32 fp32 columns
        const int slab_cols = out_bf16 ? 64 : 32;
#pragma unroll 1
        for (int col = col_begin; col < col_begin + EPI_COLS; col += slab_cols) {
          const int n = c.n0 + col;
          if (n >= p.N) break;
          uint8_t* slab = mine + (Cfg::EPI_SLABS == 2 ? (epi_round & 1) * (Cfg::EPI_WARPS * 4096) : 0);
          // the store that last read this slab must have finished reading it
          if (lane == 0) {
            if (Cfg::EPI_SLABS == 2) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            else tma_store_wait_read();
          }
          __syncwarp();
          uint8_t* rowp = slab + lane * 128;
          if (out_bf16) {
            uint32_t r0[32], r1[32];
            tmem_ld_x32(t_addr + col, r0);
            tmem_ld_x32(t_addr + col + 32, r1);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              const uint32_t* src = v < 4 ? &r0[8 * v] : &r1[8 * (v - 4)];
              uint4 q;
              if (empty_k) {
                q = make_uint4(0, 0, 0, 0);
              } else {
                q.x = pack_bf16(__uint_as_float(src[0]), __uint_as_float(src[1]));
                q.y = pack_bf16(__uint_as_float(src[2]), __uint_as_float(src[3]));
                q.z = pack_bf16(__uint_as_float(src[4]), __uint_as_float(src[5]));
                q.w = pack_bf16(__uint_as_float(src[6]), __uint_as_float(src[7]));
              }
              *reinterpret_cast<uint4*>(rowp + ((v ^ (lane & 7)) << 4)) = q;
            }
          } else {
            uint32_t r0[32];
            tmem_ld_x32(t_addr + col, r0);
            tmem_ld_wait();
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              uint4 q = empty_k ? make_uint4(0, 0, 0, 0)
                                : make_uint4(r0[4 * v], r0[4 * v + 1], r0[4 * v + 2], r0[4 * v + 3]);
              *reinterpret_cast<uint4*>(rowp + ((v ^ (lane & 7)) << 4)) = q;
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0) {
            if (out_adds) tma_reduce_add_2d(&p.tmap_c, slab, n, out_row0);   // in C's own type (fp32 or bf16)
            else tma_store_2d(&p.tmap_c, slab, n, out_row0);
            tma_store_commit();
          }
          ++epi_round;
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[acc]);
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
        continue;
      }
#pragma unroll 1
      for (int col = col_begin; col < col_begin + EPI_COLS; col += 32) {
        uint32_t r[32];
        tmem_ld_x32(t_addr + col, r);
        tmem_ld_wait();
        if (empty_k) {
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = 0;
        }
        const int n = c.n0 + col;
        if (!row_ok || n >= p.N) continue;
        const int valid = min(32, p.N - n);
        if (out_bf16 && out_adds) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + out_row * p.ldc + n;
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i < valid) dst[i] = __float2bfloat16(__bfloat162float(dst[i]) + __uint_as_float(r[i]));
        } else if (out_bf16) {
          __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.c) + out_row * p.ldc + n;
          if (valid == 32) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 q;
              q.x = pack_bf16(__uint_as_float(r[8 * v + 0]), __uint_as_float(r[8 * v + 1]));
              q.y = pack_bf16(__uint_as_float(r[8 * v + 2]), __uint_as_float(r[8 * v + 3]));
              q.z = pack_bf16(__uint_as_float(r[8 * v + 4]), __uint_as_float(r[8 * v + 5]));
              q.w = pack_bf16(__uint_as_float(r[8 * v + 6]), __uint_as_float(r[8 * v + 7]));
              reinterpret_cast<uint4*>(dst)[v] = q;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)  // unrolled with a predicate: r[] stays in registers
              if (i < valid) dst[i] = __float2bfloat16(__uint_as_float(r[i]));
          }
        } else {
          float* dst = reinterpret_cast<float*>(p.c) + out_row * p.ldc + n;
          if (valid == 32) {
#pragma unroll
            for (int v = 0; v < 8; ++v) {
              float4 q = make_float4(__uint_as_float(r[4 * v]), __uint_as_float(r[4 * v + 1]),
                                     __uint_as_float(r[4 * v + 2]), __uint_as_float(r[4 * v + 3]));
              if (p.out_kind == OUT_F32_ACC) {
                float4 o = reinterpret_cast<float4*>(dst)[v];
                q.x += o.x; q.y += o.y; q.z += o.z; q.w += o.w;
              }
              reinterpret_cast<float4*>(dst)[v] = q;
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (i < valid) {
                const float x = __uint_as_float(r[i]);
                dst[i] = p.out_kind == OUT_F32_ACC ? dst[i] + x : x;
              }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[acc]);
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1; }
    }
  }

  // ---------------------------------------------------------------- teardown
  if (warp >= 2 && lane == 0) tma_store_wait_all();  // this warp's stores have left shared memory and landed
  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // give loads that are still in flight time to land before the CTA's memory is reused
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult res;
    cudaError_t err = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &res);
    if (err != cudaSuccess || res != cudaDriverEntryPointSuccess || ptr == nullptr) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes` elements, box = box_cols x box_rows,
// 128-byte swizzle (box_cols * elem_bytes must be 128).
const char* make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows,
                         uint64_t cols, uint64_t row_stride_bytes, uint32_t box_cols,
                         uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return "cuTensorMapEncodeTiled is not available from this driver";
  // The driver call needs this thread's primary context bound; a thread that has made
  // no runtime call yet (an autograd worker) has none until one is made.
  static thread_local bool bound = false;
  if (!bound) { cudaFree(nullptr); bound = true; }
  if (reinterpret_cast<uintptr_t>(base) % 16 != 0) return "tensor base is not 16-byte aligned";
  if (row_stride_bytes % 16 != 0) return "row stride is not a multiple of 16 bytes";
  CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                         : elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r == CUDA_SUCCESS) return nullptr;
  static thread_local char msg[256];
  snprintf(msg, sizeof(msg), "cuTensorMapEncodeTiled failed (code %d): base %p elem %d dims [%llu, %llu] stride %llu box [%u, %u]",
           (int)r, base, elem_bytes, (unsigned long long)cols, (unsigned long long)rows,
           (unsigned long long)row_stride_bytes, box_cols, box_rows);
  return msg;
}

template <int KIND, int BN, bool A_MN, bool B_MN, int EW = 4>
static const char* launch_cfg(const GemmParams& p, int sms, cudaStream_t stream) {
  using Cfg = GemmCfg<KIND, BN, EW>;
  auto kern = gemm_sm100_kernel<KIND, BN, A_MN, B_MN, EW>;
  static bool configured[64] = {};
  if (!allow_dynamic_smem(kern, Cfg::SMEM_BYTES, configured))
    return "cudaFuncSetAttribute(max dynamic shared memory) failed";
  kern<<<sms, Cfg::THREADS, Cfg::SMEM_BYTES, stream>>>(p);
  return cudaGetLastError() == cudaSuccess ? nullptr : "gemm kernel launch failed";
}

const char* gemm_launch(const GemmArgs& a, cudaStream_t stream) {
  GemmParams p;
  p.mode = a.mode; p.M = a.M; p.N = a.N; p.K = a.K; p.k_total = a.k_total > 0 ? a.k_total : a.K;
  p.groups = a.groups; p.group_offsets = a.group_offsets;
  p.c = a.c; p.ldc = a.ldc; p.out_kind = a.out_kind;
  p.sfa = a.sfa; p.sfb = a.sfb; p.status = a.status;
  p.wait_flags = a.wait_flags; p.wait_world = a.wait_world; p.wait_epoch = a.wait_epoch; p.wait_limit_ns = a.wait_limit_ns;
  p.wait_rows = a.wait_rows; p.m_rotate = a.m_rotate; p.wait_on_k = a.wait_on_k ? 1 : 0; p.wait_on_n = a.wait_on_n ? 1 : 0;
  if (a.wait_world > 32) return "at most 32 senders can be waited for";
  const int elem = a.kind == KIND_BF16 ? 2 : 1;
  const int bk = a.kind == KIND_BF16 ? 64 : 128;
  const int bn = a.bn;
  if (a.kind == KIND_MXFP8 && (a.a_mn || a.b_mn)) return "mxfp8 operands are K-major";
  if (a.kind == KIND_MXFP8 && (p.k_total % 128 != 0)) return "mxfp8 K must be a multiple of 128";
  const char* err;
  // A: K-major [a_rows, K] box {bk, 128};  MN-major stored [K, a_rows] box {64, bk}
  if (a.a_mn) err = make_tmap_2d(&p.tmap_a, a.a, elem, a.a_outer, a.a_inner, a.lda_bytes, 64, bk);
  else        err = make_tmap_2d(&p.tmap_a, a.a, elem, a.a_outer, a.a_inner, a.lda_bytes, bk, BM);
  if (err) return err;
  if (a.b_mn) err = make_tmap_2d(&p.tmap_b, a.b, elem, a.b_outer, a.b_inner, a.ldb_bytes, 64, bk);
  else        err = make_tmap_2d(&p.tmap_b, a.b, elem, a.b_outer, a.b_inner, a.ldb_bytes, bk, bn);
  if (err) return err;
  p.tma_store = 0;
  const int c_elem = (a.out_kind == OUT_BF16 || a.out_kind == OUT_BF16_ACC) ? 2 : 4;
  if (a.ldc * c_elem % 16 == 0 && reinterpret_cast<uintptr_t>(a.c) % 16 == 0 &&
      (a.mode != MODE_GROUPED_K || a.M % BM == 0)) {
    // rows of C: every row the walk can touch (grouped rows: the sorted, padded row count;
    // grouped contraction: the groups' [M, N] outputs stacked). Boxes are 32 rows x 128 bytes;
    // fp32 accumulation into C is a TMA reduce-add (no read of C by the SMs).
    const uint64_t rows = a.mode == MODE_GROUPED_K ? (uint64_t)a.groups * a.M : (uint64_t)a.M;
    if (make_tmap_2d(&p.tmap_c, a.c, c_elem, rows, (uint64_t)a.N, (uint64_t)a.ldc * c_elem, 128 / c_elem, 32) == nullptr)
      p.tma_store = 1;
  }
  const int sms = a.sms > 0 ? a.sms : 148;
#define BUX_GEMM_CASE(KIND_, BN_, AMN_, BMN_) \
  if (a.kind == KIND_ && bn == BN_ && a.a_mn == AMN_ && a.b_mn == BMN_) \
    return launch_cfg<KIND_, BN_, AMN_, BMN_>(p, sms, stream);
  BUX_GEMM_CASE(KIND_BF16, 256, false, false)
  BUX_GEMM_CASE(KIND_BF16, 256, false, true)
  BUX_GEMM_CASE(KIND_BF16, 256, true, false)
  BUX_GEMM_CASE(KIND_BF16, 256, true, true)
  BUX_GEMM_CASE(KIND_BF16, 128, false, false)
  BUX_GEMM_CASE(KIND_BF16, 128, false, true)
  BUX_GEMM_CASE(KIND_BF16, 128, true, false)
  BUX_GEMM_CASE(KIND_BF16, 128, true, true)
  BUX_GEMM_CASE(KIND_MXFP8, 128, false, false)
  if (a.kind == KIND_MXFP8 && bn == 256 && a.mode == MODE_GROUPED_ROWS)
    return launch_cfg<KIND_MXFP8, 256, false, false, 8>(p, sms, stream);
  BUX_GEMM_CASE(KIND_MXFP8, 256, false, false)
#undef BUX_GEMM_CASE
  return "no gemm kernel for this configuration";
}

}  // namespace bux
