// Expert-parallel token exchange over NVLink peer memory, issued from inside kernels.
//
// Every rank maps every peer's receive buffers (symmetric memory) and holds their base
// addresses in a small device table. The exchange is then plain loads and stores:
//   ep_push_rows     each rank writes its token rows straight into the expert-sorted
//                    receive buffer of the rank that owns the expert (P2P 16-byte
//                    stores), optionally scaled (the backward sends w * dout).
//   ep_signal        after a push (stream order), publishes an epoch number in every
//                    peer's flag row with a system-scope release store.
//   ep_pull_combine  out[t] = sum_j w[t,j] * y_peer[rank(t,j)][row(t,j)]: the combine
//                    reads the expert outputs where they were produced (P2P 16-byte
//                    loads), after a bounded wait for the owners' "output ready" flags.
//   ep_pull_dot      dw[t,j] = <y_peer[rank][row], dout[t]> for the router's gradient.
// The consumer GEMM waits for the senders' flags in its TMA producer warp
// (GemmParams::wait_flags), so nothing on the host separates exchange and compute.
//
// All waits are bounded by wall-clock time; a wait that runs out records itself in the
// status word and the kernel returns. No load here is a TMA / cluster-multicast load.
//
// Reference counterparts: parallel/experts.py:256-460 (all_to_all / ragged_all_to_all)
// and the TransformerEngine NCCL-EP primitives of parallel/nccl_ep.py:359-474.
#include "comm_sm100.h"
#include "common.cuh"

namespace bux {

constexpr int KID_EP = 4;

__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Wait until flags[0..world) >= epoch. One lane per peer, bounded.
__device__ __forceinline__ bool wait_flags(const int* flags, int world, int epoch, uint64_t limit_ns,
                                           Status* st, int site) {
  bool ok = true;
  if (threadIdx.x < world) {
    const uint64_t t0 = global_ns();
    while (ld_acquire_sys(flags + threadIdx.x) < epoch) {
      if (global_ns() - t0 > limit_ns) { ok = false; report_failure(st, KID_EP, site); break; }
      __nanosleep(200);
    }
  }
  return ok;
}

// rows: one warp per sorted pick. peer_base[r] = base of rank r's receive buffer
// ([cap rows, d] bf16). dst_rank / dst_row / src_token: int32[picks]; dst_row < 0 = dropped.
__global__ void ep_push_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ src_token,
                                    const int* __restrict__ dst_rank, const int* __restrict__ dst_row,
                                    const float* __restrict__ row_scale, const uint64_t* __restrict__ peer_base,
                                    const uint64_t* __restrict__ peer_scale, long picks, int d) {
  // With `peer_scale` (the peers' fp32 [rows] buffers) a row travels as it is and its scale
  // is stored beside it on the owner, who applies it later; without, the row is scaled here.
  const int lane = threadIdx.x & 31;
  const int vec = d / 8;
  for (long i = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < picks;
       i += (long)gridDim.x * (blockDim.x >> 5)) {
    const int row = dst_row[i];
    if (row < 0) continue;
    const uint4* src = reinterpret_cast<const uint4*>(x + (long)src_token[i] * d);
    uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(peer_base[dst_rank[i]]) + (long)row * d);
    const float s = row_scale ? row_scale[i] : 1.f;
    if (peer_scale != nullptr && lane == 0) reinterpret_cast<float*>(peer_scale[dst_rank[i]])[row] = s;
    for (int c = lane; c < vec; c += 32) {
      uint4 v = src[c];
      if (row_scale && peer_scale == nullptr) {
        uint32_t* u = &v.x;
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float2 f = unpack_bf16(u[q]); u[q] = pack_bf16(f.x * s, f.y * s); }
      }
      dst[c] = v;
    }
  }
}

// The MXFP8 exchange: a token's row is read and quantised once (e4m3 bytes + E8M0 scales along
// the row) and stored into the buffer of every expert that picked it, so the owner's first GEMM
// reads what arrived without a quantiser pass in between. One warp per token; lanes 0..k-1 hold
// the picks' destinations; a warp iteration covers 1024 columns in two halves whose loads are
// both in flight before the first is used (16 bytes per lane and half, so every store
// instruction writes 512 contiguous bytes); two neighbouring lanes share a block of 32.
// The scales leave row-major ([cap, d/32] bytes, 32 contiguous bytes per row and iteration):
// in the tensor core's tile layout a row's scales are 4-byte pieces 512 bytes apart, sixteen
// small packets over NVLink where this sends one; the owner rearranges them (`sf_rows_to_tiles`).
__global__ void ep_push_rows_mx_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ rank_of,
                                       const int* __restrict__ row_of, const float* __restrict__ w,
                                       const uint64_t* __restrict__ peer_q, const uint64_t* __restrict__ peer_sf,
                                       const uint64_t* __restrict__ peer_scale, long tokens, int k, int d) {
  const int lane = threadIdx.x & 31;
  const int sf_cols = d / 32;
  for (long t = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); t < tokens;
       t += (long)gridDim.x * (blockDim.x >> 5)) {
    int my_row = -1;
    unsigned long long my_q = 0, my_sf = 0;
    if (lane < k) {
      my_row = row_of[t * k + lane];
      if (my_row >= 0) {
        const int rank = rank_of[t * k + lane];
        my_q = peer_q[rank] + (unsigned long long)my_row * d;
        my_sf = peer_sf[rank] + (unsigned long long)my_row * sf_cols;
        if (peer_scale != nullptr) reinterpret_cast<float*>(peer_scale[rank])[my_row] = w ? w[t * k + lane] : 1.f;
      }
    }
    const __nv_bfloat16* src = x + t * d;
    for (int c0 = 0; c0 < d; c0 += 1024) {
      uint4 in[2][2];
      int col[2];
      bool live[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        col[hh] = c0 + hh * 512 + lane * 16;
        live[hh] = col[hh] < d;
        in[hh][0] = in[hh][1] = make_uint4(0, 0, 0, 0);
        if (live[hh]) {
          in[hh][0] = *reinterpret_cast<const uint4*>(src + col[hh]);
          in[hh][1] = *reinterpret_cast<const uint4*>(src + col[hh] + 8);
        }
      }
      uint4 o[2];
      uint32_t word[2];   // lanes 0, 8, 16, 24: four consecutive blocks' scales of half hh
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float v[16];
        const uint32_t* au = &in[hh][0].x; const uint32_t* bu = &in[hh][1].x;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack_bf16(au[q]), g = unpack_bf16(bu[q]);
          v[2 * q] = f.x; v[2 * q + 1] = f.y; v[8 + 2 * q] = g.x; v[8 + 2 * q + 1] = g.y;
        }
        float amax = 0.f;
#pragma unroll
        for (int q = 0; q < 16; ++q) amax = fmaxf(amax, fabsf(v[q]));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));   // the block's other half
        const uint32_t e = live[hh] ? (uint32_t)e8m0_of(amax) : 127u;
        const float inv = e8m0_inv((uint8_t)e);
        o[hh].x = cvt_e4m3x4(v[0] * inv, v[1] * inv, v[2] * inv, v[3] * inv);
        o[hh].y = cvt_e4m3x4(v[4] * inv, v[5] * inv, v[6] * inv, v[7] * inv);
        o[hh].z = cvt_e4m3x4(v[8] * inv, v[9] * inv, v[10] * inv, v[11] * inv);
        o[hh].w = cvt_e4m3x4(v[12] * inv, v[13] * inv, v[14] * inv, v[15] * inv);
        word[hh] = e | (__shfl_down_sync(0xffffffffu, e, 2) << 8) | (__shfl_down_sync(0xffffffffu, e, 4) << 16) |
                   (__shfl_down_sync(0xffffffffu, e, 6) << 24);
      }
      // rows of a multiple of 512 columns: the iteration's 32 scales as two 16-byte pieces, the
      // first half's in lane 0, the second's in lane 1 (other widths store the 4-byte words)
      const bool wide = (sf_cols & 15) == 0;
      uint4 sfv = make_uint4(0, 0, 0, 0);
      if (wide) {
        const uint32_t w0 = __shfl_sync(0xffffffffu, word[0], 0), w1 = __shfl_sync(0xffffffffu, word[0], 8);
        const uint32_t w2 = __shfl_sync(0xffffffffu, word[0], 16), w3 = __shfl_sync(0xffffffffu, word[0], 24);
        const uint32_t x0 = __shfl_sync(0xffffffffu, word[1], 0), x1 = __shfl_sync(0xffffffffu, word[1], 8);
        const uint32_t x2 = __shfl_sync(0xffffffffu, word[1], 16), x3 = __shfl_sync(0xffffffffu, word[1], 24);
        sfv = (lane & 1) ? make_uint4(x0, x1, x2, x3) : make_uint4(w0, w1, w2, w3);
      }
      for (int j = 0; j < k; ++j) {
        const int row = __shfl_sync(0xffffffffu, my_row, j);
        const unsigned long long q_dst = __shfl_sync(0xffffffffu, my_q, j);
        const unsigned long long sf_dst = __shfl_sync(0xffffffffu, my_sf, j);
        if (row < 0) continue;   // a dropped pick (the same for the whole warp)
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
          if (live[hh]) *reinterpret_cast<uint4*>(q_dst + col[hh]) = o[hh];
        if (wide) {
          if (lane < 2 && c0 + lane * 512 < d) *reinterpret_cast<uint4*>(sf_dst + (c0 >> 5) + lane * 16) = sfv;
        } else if ((lane & 7) == 0) {
#pragma unroll
          for (int hh = 0; hh < 2; ++hh)
            if (live[hh]) *reinterpret_cast<uint32_t*>(sf_dst + (col[hh] >> 5)) = word[hh];
        }
      }
    }
  }
}

// one thread per peer: flag row `channel` of peer p, slot my_rank <- epoch
__global__ void ep_signal_kernel(const uint64_t* __restrict__ peer_flags, int channel, int world,
                                 int my_rank, int epoch) {
  if (threadIdx.x < world) {
    __threadfence_system();
    int* flags = reinterpret_cast<int*>(peer_flags[threadIdx.x]) + (long)channel * world;
    st_release_sys(flags + my_rank, epoch);
  }
}

// out[t] = sum_j w[t,j] * y_peer[rank][row]; waits for every peer's flag first.
__global__ void ep_pull_combine_kernel(const uint64_t* __restrict__ peer_base, const int* __restrict__ rank_of,
                                       const int* __restrict__ row_of, const float* __restrict__ w,
                                       __nv_bfloat16* __restrict__ out, long tokens, int k, int d,
                                       const int* __restrict__ flags, int world, int epoch,
                                       uint64_t limit_ns, Status* st) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (flags != nullptr) {
    if (!wait_flags(flags, world, epoch, limit_ns, st, 1)) ok_s = 0;
    __syncthreads();
    if (!ok_s) return;
  }
  const int vec = d / 8;
  const long total = tokens * vec;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / vec; const int c = (int)(i % vec);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    // the picks' rows sit on other GPUs: up to eight loads are put in flight before the first
    // one is used, so that a thread covers the link's latency once per token, not once per pick
    for (int j0 = 0; j0 < k; j0 += 8) {
      uint4 v[8];
      float ww[8];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const int j = j0 + jj;
        v[jj] = make_uint4(0, 0, 0, 0);
        ww[jj] = 0.f;
        if (j < k) {
          const int r = row_of[t * k + j];
          if (r >= 0) {
            ww[jj] = w ? w[t * k + j] : 1.f;
            v[jj] = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peer_base[rank_of[t * k + j]]) + (long)r * d)[c];
          }
        }
      }
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const uint32_t* u = &v[jj].x;
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float2 f = unpack_bf16(u[q]); acc[2 * q] += ww[jj] * f.x; acc[2 * q + 1] += ww[jj] * f.y; }
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + t * d)[c] = o;
  }
}

// dw[t,j] = <y_peer[rank][row], dout[t]>: one warp per pick
__global__ void ep_pull_dot_kernel(const uint64_t* __restrict__ peer_base, const int* __restrict__ rank_of,
                                   const int* __restrict__ row_of, const __nv_bfloat16* __restrict__ dout,
                                   float* __restrict__ dw, long picks, int k, int d) {
  const int lane = threadIdx.x & 31;
  const int vec = d / 8;
  for (long i = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < picks;
       i += (long)gridDim.x * (blockDim.x >> 5)) {
    const int r = row_of[i];
    float dot = 0.f;
    if (r >= 0) {
      const uint4* y = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(peer_base[rank_of[i]]) + (long)r * d);
      const uint4* g = reinterpret_cast<const uint4*>(dout + (i / k) * d);
      for (int c = lane; c < vec; c += 32) {
        const uint4 a = y[c], b = g[c];
        const uint32_t* au = &a.x; const uint32_t* bu = &b.x;
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float2 f = unpack_bf16(au[q]), h = unpack_bf16(bu[q]); dot += f.x * h.x + f.y * h.y; }
      }
    }
    dot = warp_sum(dot);
    if (lane == 0) dw[i] = dot;
  }
}

// out[r] = <a[r], b[r]> over rows of d bf16 (one warp per row): the owner's share of the router
// weights' gradient, from the dy rows it received and the y rows it produced.
__global__ void row_dots_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                float* __restrict__ out, long rows, int d) {
  const int lane = threadIdx.x & 31;
  const int vec = d / 8;
  for (long i = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < rows;
       i += (long)gridDim.x * (blockDim.x >> 5)) {
    const uint4* ar = reinterpret_cast<const uint4*>(a + i * d);
    const uint4* br = reinterpret_cast<const uint4*>(b + i * d);
    float dot = 0.f;
    for (int c = lane; c < vec; c += 32) {
      const uint4 x = ar[c], y = br[c];
      const uint32_t* xu = &x.x; const uint32_t* yu = &y.x;
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = unpack_bf16(xu[q]), h = unpack_bf16(yu[q]); dot += f.x * h.x + f.y * h.y; }
    }
    dot = warp_sum(dot);
    if (lane == 0) out[i] = dot;
  }
}

// out[i] = peer[rank_of[i]][row_of[i]] (fp32 scalars; 0 for dropped picks), after every peer's flag.
__global__ void ep_pull_scalar_kernel(const uint64_t* __restrict__ peer_base, const int* __restrict__ rank_of,
                                      const int* __restrict__ row_of, float* __restrict__ out, long picks,
                                      const int* __restrict__ flags, int world, int epoch, uint64_t limit_ns,
                                      Status* st) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (flags != nullptr) {
    if (!wait_flags(flags, world, epoch, limit_ns, st, 3)) ok_s = 0;
    __syncthreads();
    if (!ok_s) return;
  }
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < picks; i += (long)gridDim.x * blockDim.x) {
    const int r = row_of[i];
    out[i] = r >= 0 ? reinterpret_cast<const float*>(peer_base[rank_of[i]])[r] : 0.f;
  }
}

// Waits for flags on the stream (used where the consumer is not one of our kernels).
__global__ void ep_wait_kernel(const int* __restrict__ flags, int world, int epoch, uint64_t limit_ns, Status* st) {
  wait_flags(flags, world, epoch, limit_ns, st, 2);
}

// Row-major E8M0 scales ([rows, sf_cols] bytes, sf_cols % 4 == 0) → the tensor core's tile layout
// (512-byte tiles of 128 rows x 4 scales), one 4-byte word per thread.
__global__ void sf_rows_to_tiles_kernel(const uint32_t* __restrict__ src, uint8_t* __restrict__ dst, long rows,
                                        int sf_cols) {
  const int words = sf_cols >> 2;
  const long total = rows * words;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long row = i / words; const int j = (int)(i % words);
    *reinterpret_cast<uint32_t*>(dst + sf_offset(row, 4 * j, sf_cols)) = src[i];
  }
}

// Rows [start[g] + count[g], start[g + 1]) of each group are padding up to the GEMM tile:
// clear them so that contractions over rows (weight gradients) see zeros there.
__global__ void zero_pad_rows_kernel(__nv_bfloat16* __restrict__ buf, const int* __restrict__ offsets,
                                     const int* __restrict__ counts, int d) {
  const int g = blockIdx.x;
  const int first = offsets[g] + counts[g], last = offsets[g + 1];
  const int vec = d / 8;
  for (int r = first + blockIdx.y; r < last; r += gridDim.y)
    for (int c = threadIdx.x; c < vec; c += blockDim.x)
      reinterpret_cast<uint4*>(buf + (long)r * d)[c] = make_uint4(0, 0, 0, 0);
}

// Tensor / sequence parallelism: this rank's block of rows goes into every other rank's
// gather buffer at row `my_rank * rows`, 16 bytes per store (its own copy is a local
// copy made by the caller, which lets the GEMM start on it at once).
__global__ void tp_push_block_kernel(const uint4* __restrict__ src, const uint64_t* __restrict__ peer_base,
                                     int world, int my_rank, long vecs_per_block) {
  const long total = vecs_per_block * (world - 1);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    // peers in rotated order so the ranks do not all write to the same GPU at once
    const int step = (int)(i / vecs_per_block);
    const int peer = (my_rank + 1 + step) % world;
    const long v = i % vecs_per_block;
    uint4* dst = reinterpret_cast<uint4*>(peer_base[peer]) + (long)my_rank * vecs_per_block + v;
    *dst = src[v];
  }
}

// out[r, :] = (residual[r, :] +) sum over peers p of partial_p[my_rank * rows + r, :]: the
// reduce-scatter of row-parallel partial sums by peer loads, fp32 accumulation. Waits
// (bounded) for every peer's flag first.
__global__ void tp_pull_reduce_kernel(const uint64_t* __restrict__ peer_base, int world, int my_rank, long rows,
                                      int d, __nv_bfloat16* __restrict__ out,
                                      const __nv_bfloat16* __restrict__ residual, const int* __restrict__ flags,
                                      int epoch, uint64_t limit_ns, Status* st) {
  __shared__ int ok_s;
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if (flags != nullptr) {
    if (!wait_flags(flags, world, epoch, limit_ns, st, 3)) ok_s = 0;
    __syncthreads();
    if (!ok_s) return;
  }
  const int vec = d / 8;
  const long total = rows * vec;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (residual != nullptr) {
      const uint4 v = reinterpret_cast<const uint4*>(residual)[i];
      float2 t;
      t = unpack_bf16(v.x); acc[0] = t.x; acc[1] = t.y; t = unpack_bf16(v.y); acc[2] = t.x; acc[3] = t.y;
      t = unpack_bf16(v.z); acc[4] = t.x; acc[5] = t.y; t = unpack_bf16(v.w); acc[6] = t.x; acc[7] = t.y;
    }
    for (int s = 0; s < world; ++s) {
      const int peer = (my_rank + s) % world;
      const uint4 v = *(reinterpret_cast<const uint4*>(peer_base[peer]) + (long)my_rank * total + i);
      float2 t;
      t = unpack_bf16(v.x); acc[0] += t.x; acc[1] += t.y; t = unpack_bf16(v.y); acc[2] += t.x; acc[3] += t.y;
      t = unpack_bf16(v.z); acc[4] += t.x; acc[5] += t.y; t = unpack_bf16(v.w); acc[6] += t.x; acc[7] += t.y;
    }
    reinterpret_cast<uint4*>(out)[i] = make_uint4(pack_bf16(acc[0], acc[1]), pack_bf16(acc[2], acc[3]),
                                                  pack_bf16(acc[4], acc[5]), pack_bf16(acc[6], acc[7]));
  }
}

// CTAs per SM the exchange kernels may take (they run beside GEMMs whose CTAs need the rest)
static int g_comm_ctas_per_sm = 0;
void set_comm_ctas_per_sm(int n) { g_comm_ctas_per_sm = n; }
static inline int comm_cap(int dflt_per_sm) { return 148 * (g_comm_ctas_per_sm > 0 ? g_comm_ctas_per_sm : dflt_per_sm); }

static inline int blocks_for(long warps_needed, int warps_per_block, int cap) {
  long g = (warps_needed + warps_per_block - 1) / warps_per_block;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

void ep_push_rows(const void* x, const int* src_token, const int* dst_rank, const int* dst_row,
                  const float* row_scale, const uint64_t* peer_base, const uint64_t* peer_scale, long picks, int d,
                  int sms, cudaStream_t s) {
  // a modest number of CTAs keeps most SMs free for the GEMMs that run beside the exchange
  ep_push_rows_kernel<<<blocks_for(picks, 8, sms > 0 ? sms * 4 : comm_cap(4)), 256, 0, s>>>(
      (const __nv_bfloat16*)x, src_token, dst_rank, dst_row, row_scale, peer_base, peer_scale, picks, d);
}
void ep_push_rows_mx(const void* x, const int* rank_of, const int* row_of, const float* w, const uint64_t* peer_q,
                     const uint64_t* peer_sf, const uint64_t* peer_scale, long tokens, int k, int d, int sms,
                     cudaStream_t s) {
  ep_push_rows_mx_kernel<<<blocks_for(tokens, 8, sms > 0 ? sms * 4 : comm_cap(4)), 256, 0, s>>>(
      (const __nv_bfloat16*)x, rank_of, row_of, w, peer_q, peer_sf, peer_scale, tokens, k, d);
}
void row_dots(const void* a, const void* b, float* out, long rows, int d, cudaStream_t s) {
  row_dots_kernel<<<blocks_for(rows, 8, 148 * 8), 256, 0, s>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b, out, rows, d);
}
void ep_pull_scalar(const uint64_t* peer_base, const int* rank_of, const int* row_of, float* out, long picks,
                    const int* flags, int world, int epoch, uint64_t limit_ns, Status* st, cudaStream_t s) {
  int grid = (int)((picks + 255) / 256 > 148 * 4 ? 148 * 4 : (picks + 255) / 256);
  ep_pull_scalar_kernel<<<grid < 1 ? 1 : grid, 256, 0, s>>>(peer_base, rank_of, row_of, out, picks, flags, world, epoch,
                                                           limit_ns, st);
}
void ep_signal(const uint64_t* peer_flags, int channel, int world, int my_rank, int epoch, cudaStream_t s) {
  ep_signal_kernel<<<1, 32, 0, s>>>(peer_flags, channel, world, my_rank, epoch);
}
void ep_pull_combine(const uint64_t* peer_base, const int* rank_of, const int* row_of, const float* w, void* out,
                     long tokens, int k, int d, const int* flags, int world, int epoch, uint64_t limit_ns,
                     Status* st, cudaStream_t s) {
  long work = tokens * (d / 8);
  const int cap = comm_cap(8);
  int grid = (int)((work + 255) / 256 > cap ? cap : (work + 255) / 256);
  ep_pull_combine_kernel<<<grid < 1 ? 1 : grid, 256, 0, s>>>(peer_base, rank_of, row_of, w, (__nv_bfloat16*)out,
                                                            tokens, k, d, flags, world, epoch, limit_ns, st);
}
void ep_pull_dot(const uint64_t* peer_base, const int* rank_of, const int* row_of, const void* dout, float* dw,
                 long picks, int k, int d, cudaStream_t s) {
  ep_pull_dot_kernel<<<blocks_for(picks, 8, 148 * 8), 256, 0, s>>>(peer_base, rank_of, row_of,
                                                                    (const __nv_bfloat16*)dout, dw, picks, k, d);
}
void sf_rows_to_tiles(const void* src, void* dst, long rows, int sf_cols, cudaStream_t s) {
  const long total = rows * (sf_cols >> 2);
  int grid = (int)((total + 255) / 256 > 148 * 8 ? 148 * 8 : (total + 255) / 256);
  sf_rows_to_tiles_kernel<<<grid < 1 ? 1 : grid, 256, 0, s>>>((const uint32_t*)src, (uint8_t*)dst, rows, sf_cols);
}
void zero_pad_rows(void* buf, const int* offsets, const int* counts, int groups, int d, cudaStream_t s) {
  zero_pad_rows_kernel<<<dim3(groups, 16), 256, 0, s>>>((__nv_bfloat16*)buf, offsets, counts, d);
}
void tp_push_block(const void* src, const uint64_t* peer_base, int world, int my_rank, long rows, int d, int sms,
                   cudaStream_t s) {
  const long vecs = rows * d / 8;
  const long work = vecs * (world - 1);
  if (work <= 0) return;
  const int cap = (sms > 0 ? sms : 148) * 4;  // small CTAs without shared memory: they fit beside the GEMM's
  int grid = (int)((work + 255) / 256 > cap ? cap : (work + 255) / 256);
  tp_push_block_kernel<<<grid < 1 ? 1 : grid, 256, 0, s>>>((const uint4*)src, peer_base, world, my_rank, vecs);
}
void tp_pull_reduce(const uint64_t* peer_base, int world, int my_rank, long rows, int d, void* out,
                    const void* residual, const int* flags, int epoch, uint64_t limit_ns, Status* st,
                    cudaStream_t s) {
  const long work = rows * (d / 8);
  int grid = (int)((work + 255) / 256 > 148 * 8 ? 148 * 8 : (work + 255) / 256);
  tp_pull_reduce_kernel<<<grid < 1 ? 1 : grid, 256, 0, s>>>(peer_base, world, my_rank, rows, d, (__nv_bfloat16*)out,
                                                           (const __nv_bfloat16*)residual, flags, epoch, limit_ns, st);
}
void ep_wait(const int* flags, int world, int epoch, uint64_t limit_ns, Status* st, cudaStream_t s) {
  ep_wait_kernel<<<1, 32, 0, s>>>(flags, world, epoch, limit_ns, st);
}

}  // namespace bux
