// Causal depthwise convolution over the tokens: y[b,t,c] = sum_j w[c,j] x[b,t-j,c] (+ bias[c]),
// a tap dropped where it would reach across a document start (position[b,t] < j).
// x, y, dy, dx: [B, T, C] bf16; w: [C, taps] fp32 (taps <= 8); position: [B, T] int32 (the
// position inside its document) or null for whole rows. Memory-bound: every thread owns eight
// channels of one token (16-byte accesses, the taps' rows come from L1/L2).
// The weight gradient accumulates per thread over a slab of tokens, is summed over the block's
// token lanes in shared memory and leaves as one atomic add per (channel, tap) and block.
// Reference counterparts: architecture/layers/conv.py, architecture/recurrent/ssm.py:324.
#include "common.cuh"
#include "elementwise.h"

namespace bux {

constexpr int CONV_MAX_TAPS = 8;

template <bool BWD>
__global__ void causal_conv_kernel(const __nv_bfloat16* __restrict__ in, const float* __restrict__ w,
                                   const float* __restrict__ bias, const int* __restrict__ position,
                                   __nv_bfloat16* __restrict__ out, int B, int T, int C, int taps) {
  const int vec = C / 8;
  const long total = (long)B * T * vec;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int c8 = (int)(i % vec);
    const long bt = i / vec;
    const int t = (int)(bt % T);
    const long row0 = bt - t;            // first token of the row
    float acc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[e] = (!BWD && bias != nullptr) ? bias[c8 * 8 + e] : 0.f;
    for (int j = 0; j < taps; ++j) {
      // forward: y[t] takes x[t-j] if position[t] >= j; backward: dx[t] takes dy[t+j] if position[t+j] >= j
      const int src = BWD ? t + j : t - j;
      if (src < 0 || src >= T) continue;
      const int gate_at = BWD ? src : t;
      const int p = position ? position[row0 + gate_at] : gate_at;
      if (p < j) continue;
      const uint4 v = *reinterpret_cast<const uint4*>(in + (row0 + src) * C + c8 * 8);
      const uint32_t* u = &v.x;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = unpack_bf16(u[q]);
        acc[2 * q] += w[(c8 * 8 + 2 * q) * taps + j] * f.x;
        acc[2 * q + 1] += w[(c8 * 8 + 2 * q + 1) * taps + j] * f.y;
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + bt * C + c8 * 8) = o;
  }
}

// dw[c, j] += sum_{b,t} dy[b,t,c] x[b,t-j,c] (same gate as the forward); db[c] += sum dy[b,t,c].
// Block: 32 channel groups of 8 x 8 token lanes; grid.x over channel groups, grid.y over slabs of tokens.
__global__ void causal_conv_wgrad_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                         const int* __restrict__ position, float* __restrict__ dw,
                                         float* __restrict__ db, int B, int T, int C, int taps) {
  __shared__ float part[8][32][8];   // [token lane][channel group][channel]
  const int cg = threadIdx.x & 31, lane_t = threadIdx.x >> 5;
  const int c8 = blockIdx.x * 32 + cg;
  const bool live = c8 * 8 < C;
  const long rows = (long)B * T;
  float acc[CONV_MAX_TAPS][8], accb[8];
#pragma unroll
  for (int j = 0; j < CONV_MAX_TAPS; ++j)
#pragma unroll
    for (int e = 0; e < 8; ++e) acc[j][e] = 0.f;
#pragma unroll
  for (int e = 0; e < 8; ++e) accb[e] = 0.f;
  if (live) {
    for (long r = (long)blockIdx.y * 8 + lane_t; r < rows; r += (long)gridDim.y * 8) {
      const int t = (int)(r % T);
      const int p = position ? position[r] : t;
      const uint4 g = *reinterpret_cast<const uint4*>(dy + r * C + c8 * 8);
      float gf[8];
      {
        const uint32_t* u = &g.x;
#pragma unroll
        for (int q = 0; q < 4; ++q) { const float2 f = unpack_bf16(u[q]); gf[2 * q] = f.x; gf[2 * q + 1] = f.y; }
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) accb[e] += gf[e];
#pragma unroll
      for (int j = 0; j < CONV_MAX_TAPS; ++j) {
        if (j >= taps || t - j < 0 || p < j) continue;
        const uint4 v = *reinterpret_cast<const uint4*>(x + (r - j) * C + c8 * 8);
        const uint32_t* u = &v.x;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = unpack_bf16(u[q]);
          acc[j][2 * q] += gf[2 * q] * f.x;
          acc[j][2 * q + 1] += gf[2 * q + 1] * f.y;
        }
      }
    }
  }
  // sum over the block's eight token lanes, one quantity at a time
  for (int j = 0; j <= taps; ++j) {   // j == taps: the bias
    __syncthreads();
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float v = accb[e];
#pragma unroll
      for (int jj = 0; jj < CONV_MAX_TAPS; ++jj) if (j < taps && jj == j) v = acc[jj][e];
      part[lane_t][cg][e] = v;
    }
    __syncthreads();
    if (lane_t == 0 && live) {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float sum = 0.f;
#pragma unroll
        for (int l = 0; l < 8; ++l) sum += part[l][cg][e];
        if (j < taps) atomicAdd(&dw[(c8 * 8 + e) * taps + j], sum);
        else if (db != nullptr) atomicAdd(&db[c8 * 8 + e], sum);
      }
    }
  }
}

const char* causal_conv(bool bwd, const void* in, const float* w, const float* bias, const int* position, void* out,
                        int B, int T, int C, int taps, cudaStream_t s) {
  if (C % 8 != 0) return "causal_conv: channels must be a multiple of 8";
  if (taps < 1 || taps > CONV_MAX_TAPS) return "causal_conv: 1 to 8 taps";
  const long total = (long)B * T * (C / 8);
  const int grid = (int)((total + 255) / 256 > 148L * 16 ? 148L * 16 : (total + 255) / 256);
  if (bwd)
    causal_conv_kernel<true><<<grid < 1 ? 1 : grid, 256, 0, s>>>((const __nv_bfloat16*)in, w, nullptr, position,
                                                                  (__nv_bfloat16*)out, B, T, C, taps);
  else
    causal_conv_kernel<false><<<grid < 1 ? 1 : grid, 256, 0, s>>>((const __nv_bfloat16*)in, w, bias, position,
                                                                   (__nv_bfloat16*)out, B, T, C, taps);
  return cudaGetLastError() == cudaSuccess ? nullptr : "causal_conv launch failed";
}

const char* causal_conv_wgrad(const void* x, const void* dy, const int* position, float* dw, float* db, int B, int T,
                              int C, int taps, cudaStream_t s) {
  if (C % 8 != 0) return "causal_conv: channels must be a multiple of 8";
  if (taps < 1 || taps > CONV_MAX_TAPS) return "causal_conv: 1 to 8 taps";
  const long rows = (long)B * T;
  const int gx = (C / 8 + 31) / 32;
  long gy = (rows + 63) / 64;            // at least eight tokens per lane
  const long cap = (148L * 8 + gx - 1) / gx;
  if (gy > cap) gy = cap;
  if (gy < 1) gy = 1;
  causal_conv_wgrad_kernel<<<dim3(gx, (unsigned)gy), 256, 0, s>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                                  position, dw, db, B, T, C, taps);
  return cudaGetLastError() == cudaSuccess ? nullptr : "causal_conv wgrad launch failed";
}

}  // namespace bux
