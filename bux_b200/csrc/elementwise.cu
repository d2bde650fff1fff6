// Memory-bound kernels for sm_100a: RMSNorm (+ per-head QK-norm with RoPE), gated
// activations, the dual-orientation MXFP8 quantiser, cross-entropy over a logits
// chunk, flat AdamW (fp32 / bf16 / block-scaled 8-bit moments), and the MoE row
// gather / weighted combine. All use 128-bit accesses and fp32 math; none allocates.
//
// Reference counterparts: norm_rope Pallas kernel (architecture/attention/norm_rope.py),
// MXFP8 quantiser (architecture/precision/blockscaled.py:386-445), chunked
// cross-entropy (architecture/logits.py:209-353), optax AdamW (train/optim.py:403),
// token_rows / token_sums (architecture/experts/moe.py:992-1071).
#include "common.cuh"
#include "elementwise.h"

#include <cuda_fp4.h>

namespace bux {

// ---------------------------------------------------------------- RMSNorm
// One warp per row. x, y: [rows, d] bf16; w: [d] fp32 or null; rstd: [rows] fp32 out.
template <int VEC>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                   int rows, int d, float eps) {
  const int warps_per_block = blockDim.x >> 5;
  const int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * d);
  const int nvec = d / 8;
  float ss = 0.f;
  for (int i = lane; i < nvec; i += 32) {
    uint4 v = xr[i];
    float2 a = unpack_bf16(v.x), b = unpack_bf16(v.y), c = unpack_bf16(v.z), e = unpack_bf16(v.w);
    ss += a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y + c.x * c.x + c.y * c.y + e.x * e.x + e.y * e.y;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / d + eps);
  if (lane == 0 && rstd) rstd[row] = r;
  uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * d);
  for (int i = lane; i < nvec; i += 32) {
    uint4 v = xr[i];
    float f[8];
    float2 t;
    t = unpack_bf16(v.x); f[0] = t.x; f[1] = t.y;
    t = unpack_bf16(v.y); f[2] = t.x; f[3] = t.y;
    t = unpack_bf16(v.z); f[4] = t.x; f[5] = t.y;
    t = unpack_bf16(v.w); f[6] = t.x; f[7] = t.y;
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * r * (w ? w[i * 8 + j] : 1.f);
    uint4 o;
    o.x = pack_bf16(f[0], f[1]); o.y = pack_bf16(f[2], f[3]);
    o.z = pack_bf16(f[4], f[5]); o.w = pack_bf16(f[6], f[7]);
    yr[i] = o;
  }
}

// Backward: dx = r * (w*dy) - x * r^3 * mean(w*dy*x); dw += sum_rows dy * x * r.
// Each block walks rows grid-stride, keeps its dw partial in shared memory (fp32) and
// adds it to the global fp32 dw once at the end.
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                                   int rows, int d) {
  extern __shared__ float dw_part[];
  for (int i = threadIdx.x; i < d; i += blockDim.x) dw_part[i] = 0.f;
  __syncthreads();
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nvec = d / 8;
  for (int row = blockIdx.x * warps_per_block + warp; row < rows; row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * d);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * d);
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < nvec; i += 32) {
      uint4 xv = xr[i], gv = gr[i];
      const uint32_t* xu = &xv.x; const uint32_t* gu = &gv.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 a = unpack_bf16(xu[j]), g = unpack_bf16(gu[j]);
        const float w0 = w ? w[i * 8 + 2 * j] : 1.f, w1 = w ? w[i * 8 + 2 * j + 1] : 1.f;
        dot += a.x * g.x * w0 + a.y * g.y * w1;
      }
    }
    dot = warp_sum(dot);
    const float c = dot * r * r * r / d;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * d);
    for (int i = lane; i < nvec; i += 32) {
      uint4 xv = xr[i], gv = gr[i], o;
      const uint32_t* xu = &xv.x; const uint32_t* gu = &gv.x; uint32_t* ou = &o.x;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 a = unpack_bf16(xu[j]), g = unpack_bf16(gu[j]);
        const int col = i * 8 + 2 * j;
        const float w0 = w ? w[col] : 1.f, w1 = w ? w[col + 1] : 1.f;
        ou[j] = pack_bf16(r * w0 * g.x - a.x * c, r * w1 * g.y - a.y * c);
        if (dw) {
          atomicAdd(&dw_part[col], g.x * a.x * r);
          atomicAdd(&dw_part[col + 1], g.y * a.y * r);
        }
      }
      dxr[i] = o;
    }
  }
  __syncthreads();
  if (dw)
    for (int i = threadIdx.x; i < d; i += blockDim.x) atomicAdd(&dw[i], dw_part[i]);
}

// The same backward with one private fp32 slab of dw per warp in shared memory: a lane owns
// its columns of the slab, so the per-row update is a plain vector read-modify-write (no
// atomics); the slabs are summed once at the end. Needs 8 warps · d · 4 bytes of shared memory.
__global__ void __launch_bounds__(256)
rmsnorm_bwd_slab_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                        const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, int rows, int d) {
  extern __shared__ __align__(16) float slabs[];  // [warps][d]
  const int warps_per_block = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < warps_per_block * d; i += blockDim.x) slabs[i] = 0.f;
  __syncthreads();
  float4* mine = reinterpret_cast<float4*>(slabs + (size_t)warp * d);
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const int nvec = d / 8;
  for (int row = blockIdx.x * warps_per_block + warp; row < rows; row += gridDim.x * warps_per_block) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * d);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + (size_t)row * d);
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < nvec; i += 32) {
      const uint4 xv = xr[i], gv = gr[i];
      const uint32_t* xu = &xv.x; const uint32_t* gu = &gv.x;
      float wl[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
      if (w) {
        const float4 lo = w4[2 * i], hi = w4[2 * i + 1];
        wl[0] = lo.x; wl[1] = lo.y; wl[2] = lo.z; wl[3] = lo.w; wl[4] = hi.x; wl[5] = hi.y; wl[6] = hi.z; wl[7] = hi.w;
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = unpack_bf16(xu[j]), g = unpack_bf16(gu[j]);
        dot += a.x * g.x * wl[2 * j] + a.y * g.y * wl[2 * j + 1];
      }
    }
    dot = warp_sum(dot);
    const float c = dot * r * r * r / d;
    uint4* dxr = reinterpret_cast<uint4*>(dx + (size_t)row * d);
    for (int i = lane; i < nvec; i += 32) {
      const uint4 xv = xr[i], gv = gr[i];  // second read of the row: L1 / L2
      const uint32_t* xu = &xv.x; const uint32_t* gu = &gv.x;
      float wl[8] = {1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f, 1.f};
      if (w) {
        const float4 lo = w4[2 * i], hi = w4[2 * i + 1];
        wl[0] = lo.x; wl[1] = lo.y; wl[2] = lo.z; wl[3] = lo.w; wl[4] = hi.x; wl[5] = hi.y; wl[6] = hi.z; wl[7] = hi.w;
      }
      uint4 o; uint32_t* ou = &o.x;
      float p[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 a = unpack_bf16(xu[j]), g = unpack_bf16(gu[j]);
        ou[j] = pack_bf16(r * wl[2 * j] * g.x - a.x * c, r * wl[2 * j + 1] * g.y - a.y * c);
        p[2 * j] = g.x * a.x * r;
        p[2 * j + 1] = g.y * a.y * r;
      }
      dxr[i] = o;
      if (dw) {
        float4 lo = mine[2 * i], hi = mine[2 * i + 1];
        lo.x += p[0]; lo.y += p[1]; lo.z += p[2]; lo.w += p[3];
        hi.x += p[4]; hi.y += p[5]; hi.z += p[6]; hi.w += p[7];
        mine[2 * i] = lo; mine[2 * i + 1] = hi;
      }
    }
  }
  __syncthreads();
  if (dw)
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
      float total = 0.f;
      for (int k = 0; k < warps_per_block; ++k) total += slabs[(size_t)k * d + i];
      atomicAdd(&dw[i], total);
    }
}

// ---------------------------------------------------------------- QK-norm + RoPE
// x: [tokens, heads, D] bf16 (row stride `stride_tok` elements so it may be a slice of
// a fused qkv buffer); cos/sin: [tokens, D/2] fp32; w: [D] fp32 or null (no norm).
// One warp per (token, head): lane l holds D/32 consecutive elements; its rotation
// partner (element i <-> i + D/2) lives in lane l ^ 16.
// E consecutive bf16 (E = 2, 4 or 8: one 4-, 8- or 16-byte access; the address is a multiple
// of E elements because head offsets and token strides are multiples of the head dim).
template <int E> struct BfVec;
template <> struct BfVec<2> { using T = uint32_t; };
template <> struct BfVec<4> { using T = uint2; };
template <> struct BfVec<8> { using T = uint4; };
template <int E>
__device__ __forceinline__ void load_bf16(const __nv_bfloat16* p, float (&out)[E]) {
  const typename BfVec<E>::T raw = *reinterpret_cast<const typename BfVec<E>::T*>(p);
  const uint32_t* u = reinterpret_cast<const uint32_t*>(&raw);
#pragma unroll
  for (int j = 0; j < E / 2; ++j) { const float2 t = unpack_bf16(u[j]); out[2 * j] = t.x; out[2 * j + 1] = t.y; }
}
template <int E>
__device__ __forceinline__ void store_bf16(__nv_bfloat16* p, const float (&v)[E]) {
  typename BfVec<E>::T raw;
  uint32_t* u = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
  for (int j = 0; j < E / 2; ++j) u[j] = pack_bf16(v[2 * j], v[2 * j + 1]);
  *reinterpret_cast<typename BfVec<E>::T*>(p) = raw;
}
template <int E>
__device__ __forceinline__ void load_f32(const float* p, float (&out)[E]) {
  if (E % 4 == 0) {
#pragma unroll
    for (int j = 0; j < E / 4; ++j) {
      const float4 t = reinterpret_cast<const float4*>(p)[j];
      out[4 * j] = t.x; out[4 * j + 1] = t.y; out[4 * j + 2] = t.z; out[4 * j + 3] = t.w;
    }
  } else {
    const float2 t = *reinterpret_cast<const float2*>(p);
    out[0] = t.x; out[1] = t.y;
  }
}

template <int D, bool BWD>
__global__ void norm_rope_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                 const float* __restrict__ cs, const float* __restrict__ sn,
                                 __nv_bfloat16* __restrict__ y, float* __restrict__ rstd_io,
                                 const __nv_bfloat16* __restrict__ dy, float* __restrict__ dw,
                                 long tokens, int heads, long stride_tok_x, long stride_tok_y,
                                 float eps) {
  // D/8 lanes per (token, head), eight elements (one 16-byte access) per lane: a warp works
  // on 256/D items at once. Element i rotates with i + D/2, which lane ^ (LPI/2) holds.
  constexpr int E = 8;
  constexpr int LPI = D / E;          // lanes per item: 8, 16 or 32
  constexpr int IPW = 32 / LPI;       // items per warp
  __shared__ float dw_part[D];
  if (BWD) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) dw_part[i] = 0.f;
    __syncthreads();
  }
  const int lane = threadIdx.x & 31;
  const int sub = lane / LPI, li = lane % LPI;  // which of the warp's items, and the lane within it
  const long nwarps = (long)gridDim.x * (blockDim.x >> 5);
  const long total = tokens * heads;
  const long steps = (total + IPW - 1) / IPW;   // whole warps iterate together (shuffles stay converged)
  float dw_lane[E];  // a lane always holds the same E columns: its share of dw stays in registers
#pragma unroll
  for (int j = 0; j < E; ++j) dw_lane[j] = 0.f;
  float wl[E];
#pragma unroll
  for (int j = 0; j < E; ++j) wl[j] = w ? w[li * E + j] : 1.f;
  for (long step = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); step < steps; step += nwarps) {
    const long item = step * IPW + sub;
    const bool live = item < total;
    const long tok = live ? item / heads : 0;
    const int head = live ? (int)(item % heads) : 0;
    const __nv_bfloat16* xp = x + tok * stride_tok_x + (long)head * D + li * E;
    float v[E];
    load_bf16<E>(xp, v);
    const bool upper = li >= LPI / 2;
    const int half_idx = (li % (LPI / 2)) * E;  // index into cos/sin of my first element
    float c[E], s[E];
    load_f32<E>(cs + tok * (D / 2) + half_idx, c);
    load_f32<E>(sn + tok * (D / 2) + half_idx, s);
    if (!BWD) {
      if (w) {
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < E; ++j) ss += v[j] * v[j];
#pragma unroll
        for (int o = LPI / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float r = rsqrtf(ss / D + eps);
        if (li == 0 && live && rstd_io) rstd_io[item] = r;
#pragma unroll
        for (int j = 0; j < E; ++j) v[j] = v[j] * r * wl[j];
      }
      float out[E];
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, v[j], LPI / 2);
        // lower half: a*c - b*s ; upper half: a*s + b*c  (a = lower, b = upper element)
        out[j] = upper ? (other * s[j] + v[j] * c[j]) : (v[j] * c[j] - other * s[j]);
      }
      if (live) store_bf16<E>(y + tok * stride_tok_y + (long)head * D + li * E, out);
    } else {
      // dy -> d(normed) by the inverse rotation, then RMSNorm backward per head
      float g[E];
      load_bf16<E>(dy + tok * stride_tok_y + (long)head * D + li * E, g);
#pragma unroll
      for (int j = 0; j < E; ++j) {
        const float other = __shfl_xor_sync(0xffffffffu, g[j], LPI / 2);
        // y_lo = a c - b s, y_hi = a s + b c  =>  da = g_lo c + g_hi s, db = -g_lo s + g_hi c
        g[j] = upper ? (-other * s[j] + g[j] * c[j]) : (g[j] * c[j] + other * s[j]);
      }
      __nv_bfloat16* dxp = y + tok * stride_tok_y + (long)head * D + li * E;  // y doubles as dx (dense, like dy)
      if (w) {
        const float r = rstd_io[live ? item : 0];
        float dot = 0.f;
#pragma unroll
        for (int j = 0; j < E; ++j) dot += g[j] * wl[j] * v[j];
#pragma unroll
        for (int o = LPI / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float cc = dot * r * r * r / D;
        float o8[E];
#pragma unroll
        for (int j = 0; j < E; ++j) {
          if (live) dw_lane[j] += g[j] * v[j] * r;
          o8[j] = r * wl[j] * g[j] - v[j] * cc;
        }
        if (live) store_bf16<E>(dxp, o8);
      } else if (live) {
        store_bf16<E>(dxp, g);
      }
    }
  }
  if (BWD && dw) {
#pragma unroll
    for (int j = 0; j < E; ++j) atomicAdd(&dw_part[li * E + j], dw_lane[j]);
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&dw[i], dw_part[i]);
  }
}

// ---------------------------------------------------------------- gated activations
__device__ __forceinline__ float act_fwd(float g, int kind) {
  if (kind == ACT_SWISH) return __fdividef(g, 1.f + __expf(-g));
  if (kind == ACT_QUICK_GELU) return __fdividef(g, 1.f + __expf(-1.702f * g));
  if (kind == ACT_GELU_TANH) {
    const float u = 0.7978845608f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.f + tanhf(u));
  }
  if (kind == ACT_RELU2) { const float r = fmaxf(g, 0.f); return r * r; }
  return g;
}
__device__ __forceinline__ float act_grad(float g, int kind) {
  if (kind == ACT_SWISH) { const float s = __fdividef(1.f, 1.f + __expf(-g)); return s * (1.f + g * (1.f - s)); }
  if (kind == ACT_QUICK_GELU) { const float s = __fdividef(1.f, 1.f + __expf(-1.702f * g)); return s * (1.f + 1.702f * g * (1.f - s)); }
  if (kind == ACT_GELU_TANH) {
    const float u = 0.7978845608f * (g + 0.044715f * g * g * g);
    const float t = tanhf(u);
    return 0.5f * (1.f + t) + 0.5f * g * (1.f - t * t) * 0.7978845608f * (1.f + 3.f * 0.044715f * g * g);
  }
  if (kind == ACT_RELU2) return 2.f * fmaxf(g, 0.f);
  return 1.f;
}

// act(g) and act'(g) together: the sigmoid kinds share their one exponential and reciprocal.
__device__ __forceinline__ void act_both(float g, int kind, float& a, float& da) {
  if (kind == ACT_SWISH || kind == ACT_QUICK_GELU) {
    const float k = kind == ACT_SWISH ? 1.f : 1.702f;
    const float s = __fdividef(1.f, 1.f + __expf(-k * g));
    a = g * s;
    da = s * (1.f + k * g * (1.f - s));
    return;
  }
  a = act_fwd(g, kind);
  da = act_grad(g, kind);
}

// h: [rows, 2f] (gate columns [0,f), up columns [f,2f)); out: [rows, f].
// limit > 0 clamps gate from above and up to [-limit, limit] (gpt-oss); up_offset is
// added to up after the clamp. Optional row scale (router weight) multiplies the output.
__global__ void glu_fwd_kernel(const __nv_bfloat16* __restrict__ h, __nv_bfloat16* __restrict__ out,
                               const float* __restrict__ row_scale, long rows, int f, int kind,
                               float limit, float up_offset) {
  const long total = rows * (long)(f / 8);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long row = i / (f / 8);
    const int c8 = (int)(i % (f / 8));
    const uint4 gv = *reinterpret_cast<const uint4*>(h + row * 2 * f + c8 * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(h + row * 2 * f + f + c8 * 8);
    const float rs = row_scale ? row_scale[row] : 1.f;
    uint4 o; uint32_t* ou = &o.x; const uint32_t* gu = &gv.x; const uint32_t* uu = &uv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 g = unpack_bf16(gu[j]), u = unpack_bf16(uu[j]);
      if (limit > 0.f) {
        g.x = fminf(g.x, limit); g.y = fminf(g.y, limit);
        u.x = fminf(fmaxf(u.x, -limit), limit); u.y = fminf(fmaxf(u.y, -limit), limit);
      }
      ou[j] = pack_bf16(act_fwd(g.x, kind) * (u.x + up_offset) * rs, act_fwd(g.y, kind) * (u.y + up_offset) * rs);
    }
    *reinterpret_cast<uint4*>(out + row * f + c8 * 8) = o;
  }
}

// dh: [rows, 2f] from dout [rows, f]; with row_scale also emits d(row_scale) [rows]
// (accumulated with atomics) = sum_cols dout * act(g) * (u + off).
__global__ void glu_bwd_kernel(const __nv_bfloat16* __restrict__ h, const __nv_bfloat16* __restrict__ dout,
                               __nv_bfloat16* __restrict__ dh, const float* __restrict__ row_scale,
                               float* __restrict__ d_row_scale, long rows, int f, int kind,
                               float limit, float up_offset) {
  const long total = rows * (long)(f / 8);
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long row = i / (f / 8);
    const int c8 = (int)(i % (f / 8));
    const uint4 gv = *reinterpret_cast<const uint4*>(h + row * 2 * f + c8 * 8);
    const uint4 uv = *reinterpret_cast<const uint4*>(h + row * 2 * f + f + c8 * 8);
    const uint4 dv = *reinterpret_cast<const uint4*>(dout + row * f + c8 * 8);
    const float rs = row_scale ? row_scale[row] : 1.f;
    uint4 og, ou4; uint32_t* ogu = &og.x; uint32_t* ouu = &ou4.x;
    const uint32_t* gu = &gv.x; const uint32_t* uu = &uv.x; const uint32_t* du = &dv.x;
    float ds = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 g = unpack_bf16(gu[j]), u = unpack_bf16(uu[j]), d = unpack_bf16(du[j]);
      float gx[2] = {g.x, g.y}, ux[2] = {u.x, u.y}, dx[2] = {d.x, d.y}, rg[2], ru[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        bool g_pass = true, u_pass = true;
        float gg = gx[e], uu_ = ux[e];
        if (limit > 0.f) {
          if (gg > limit) { gg = limit; g_pass = false; }
          if (uu_ > limit) { uu_ = limit; u_pass = false; }
          if (uu_ < -limit) { uu_ = -limit; u_pass = false; }
        }
        float a, da;
        act_both(gg, kind, a, da);
        ds += dx[e] * a * (uu_ + up_offset);
        const float dsc = dx[e] * rs;
        rg[e] = g_pass ? dsc * (uu_ + up_offset) * da : 0.f;
        ru[e] = u_pass ? dsc * a : 0.f;
      }
      ogu[j] = pack_bf16(rg[0], rg[1]);
      ouu[j] = pack_bf16(ru[0], ru[1]);
    }
    *reinterpret_cast<uint4*>(dh + row * 2 * f + c8 * 8) = og;
    *reinterpret_cast<uint4*>(dh + row * 2 * f + f + c8 * 8) = ou4;
    if (d_row_scale) atomicAdd(&d_row_scale[row], ds);
  }
}

// ---------------------------------------------------------------- MXFP8 quantiser
// Tile: 128 rows x 128 columns per block of 256 threads, staged once in shared memory as
// bf16 (row pitch 272 bytes: 16-byte accesses of 8 consecutive rows hit 8 different bank
// groups). Each tile fills exactly one 512-byte scale tile of the row-wise output and one
// of the transposed output, written as whole tiles (padding scales included), and every
// byte of both quantised outputs inside the padded extents, so the caller allocates
// without clearing. Optional row gather (`row_index[r]` = source row of output row r,
// negative = zero row) fuses the MoE permute into the quantiser.
//   q_row [R, C] e4m3, sf_row tiles over (R, C/32);  q_col [C, R_pad] e4m3 (R_pad = ld_col),
//   sf_col tiles over (C, R_pad/32).
constexpr int QT = 128;
// The 128×128 bf16 tile sits in shared memory without padding, its 16-byte chunks (8 columns)
// XOR-swizzled by the row, so that three access patterns are all free of bank conflicts:
// eight consecutive chunks of a row (the load), one chunk of eight consecutive rows (the
// row-wise pass) and one chunk of rows {8a + 2m + b} (the transposing ldmatrix of the column pass).
__device__ __forceinline__ int qtile_at(int row, int chunk) {
  const int g = ((((row >> 3) ^ (row >> 1)) & 3) << 1) | (row & 1);
  return row * QT + ((chunk ^ g) << 3);
}


// What the quantiser reads its 128×128 tile from: the matrix itself, or a gated activation
// computed on the way in (the activation, or its gradient, is then never written as bf16).
#ifndef QUANT_CTAS
#define QUANT_CTAS 5
#endif
enum { QSRC_PLAIN = 0, QSRC_GLU_FWD = 1, QSRC_GLU_BWD = 2, QSRC_MX = 3 };
struct QuantGlu {
  const float* row_scale;     // PLAIN: output row r is its source row times row_scale[r] (rounded to bf16);
                              // GLU_FWD: the activation of row r times row_scale[r] (as glu_fwd_kernel)
  const __nv_bfloat16* dout;  // GLU_BWD: gradient of the activation's output [rows, f]
  int f;                      // h is [rows, 2f]: gate columns, then up columns
  int kind;
  float limit, up_offset;
  const uint8_t* src_sf;      // MX: the source is e4m3 bytes [rows, cols] with these scale tiles (along cols)
};

// Eight bf16 values of eight e4m3 bytes times their block's scale 2^(e - 127) (exact in bf16).
__device__ __forceinline__ uint4 dequant_e4m3x8(uint2 q, uint8_t e) {
  const float sc = e > 0 ? __uint_as_float((uint32_t)e << 23) : __uint_as_float(0x00400000u);
  uint4 o; uint32_t* ou = &o.x;
  const uint32_t w[2] = {q.x, q.y};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const __nv_fp8x2_storage_t pair = (__nv_fp8x2_storage_t)((w[j >> 1] >> (16 * (j & 1))) & 0xffffu);
    const float2 f = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(pair, __NV_E4M3)));
    ou[j] = pack_bf16(f.x * sc, f.y * sc);
  }
  return o;
}

// Eight gated activations from eight gates and ups (same rounding as glu_fwd_kernel).
__device__ __forceinline__ uint4 glu_fwd8(const uint4& gv, const uint4& uv, const QuantGlu& gp, float rs) {
  uint4 o; uint32_t* ou = &o.x; const uint32_t* gu = &gv.x; const uint32_t* uu = &uv.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float2 g = unpack_bf16(gu[j]), u = unpack_bf16(uu[j]);
    if (gp.limit > 0.f) {
      g.x = fminf(g.x, gp.limit); g.y = fminf(g.y, gp.limit);
      u.x = fminf(fmaxf(u.x, -gp.limit), gp.limit); u.y = fminf(fmaxf(u.y, -gp.limit), gp.limit);
    }
    ou[j] = pack_bf16(act_fwd(g.x, gp.kind) * (u.x + gp.up_offset) * rs,
                      act_fwd(g.y, gp.kind) * (u.y + gp.up_offset) * rs);
  }
  return o;
}
// Eight gradients of the gate (up_half false) or of the up (true) columns (as glu_bwd_kernel).
__device__ __forceinline__ uint4 glu_bwd8(const uint4& gv, const uint4& uv, const uint4& dv, bool up_half,
                                          const QuantGlu& gp) {
  uint4 o; uint32_t* ou = &o.x;
  const uint32_t* gu = &gv.x; const uint32_t* uu = &uv.x; const uint32_t* du = &dv.x;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 g = unpack_bf16(gu[j]), u = unpack_bf16(uu[j]), d = unpack_bf16(du[j]);
    const float gx[2] = {g.x, g.y}, ux[2] = {u.x, u.y}, dx[2] = {d.x, d.y};
    float r[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      bool g_pass = true, u_pass = true;
      float gg = gx[e], uu_ = ux[e];
      if (gp.limit > 0.f) {
        if (gg > gp.limit) { gg = gp.limit; g_pass = false; }
        if (uu_ > gp.limit) { uu_ = gp.limit; u_pass = false; }
        if (uu_ < -gp.limit) { uu_ = -gp.limit; u_pass = false; }
      }
      float a, da;
      act_both(gg, gp.kind, a, da);
      if (up_half) r[e] = u_pass ? dx[e] * a : 0.f;
      else r[e] = g_pass ? dx[e] * (uu_ + gp.up_offset) * da : 0.f;
    }
    ou[j] = pack_bf16(r[0], r[1]);
  }
  return o;
}

template <int SRC>
__global__ void __launch_bounds__(256, QUANT_CTAS)
quant_mxfp8_kernel(const __nv_bfloat16* __restrict__ x, long ld_x,
                   const int* __restrict__ row_index,
                   uint8_t* __restrict__ q_row, uint8_t* __restrict__ sf_row,
                   uint8_t* __restrict__ q_col, uint8_t* __restrict__ sf_col,
                   long rows, int cols, long ld_col, long x_batch_stride, QuantGlu gp) {
  // Registers are kept low (values are re-read from the shared tile rather than held) so
  // that six blocks fit an SM: the kernel is a stream, and blocks in flight hide its latency.
  __shared__ __align__(128) __nv_bfloat16 tile[QT * QT];
  __shared__ __align__(16) uint8_t sfr[512];
  __shared__ __align__(16) uint8_t sfc[512];
  const int sf_cols_row = ((cols / 32) + 3) & ~3;
  const int sf_cols_col = (int)(((ld_col / 32) + 3) & ~3L);
  if (blockIdx.z > 0) {
    // batched: matrix z of a stack, every output advanced by its own size
    const long z = blockIdx.z;
    x += z * x_batch_stride;
    if (q_row) { q_row += z * rows * cols; sf_row += z * ((rows + 127) / 128) * (sf_cols_row / 4) * 512; }
    if (q_col) { q_col += z * (long)cols * ld_col; sf_col += z * ((cols + 127) / 128) * (sf_cols_col / 4) * 512; }
  }
  const int tid = threadIdx.x;
  const long r0 = (long)blockIdx.y * QT;
  const int c0 = blockIdx.x * QT;
  const int cc = (tid & 15) * 8;  // load: 16 threads per row (8 elements each), 16 rows per pass
  if (SRC == QSRC_MX) {
    // the source is already MXFP8 along its columns (what a peer pushed): dequantise into the
    // tile; the column pass below then quantises along the rows
    const uint8_t* x8 = reinterpret_cast<const uint8_t*>(x);
    const int src_sf_cols = ((cols / 32) + 3) & ~3;
#pragma unroll
    for (int base = 0; base < 8; ++base) {
      const long r = r0 + base * 16 + (tid >> 4);
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < rows && c0 + cc < cols) {
        const uint2 q = *reinterpret_cast<const uint2*>(x8 + r * ld_x + c0 + cc);
        v = dequant_e4m3x8(q, gp.src_sf[sf_offset(r, (c0 + cc) >> 5, src_sf_cols)]);
      }
      *reinterpret_cast<uint4*>(&tile[qtile_at(base * 16 + (tid >> 4), tid & 15)]) = v;
    }
  } else if (SRC == QSRC_PLAIN) {
#pragma unroll
    for (int base = 0; base < 8; base += 4) {
      uint4 v[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const long r = r0 + (base + i) * 16 + (tid >> 4);
        long src = r;
        if (row_index && r < rows) src = row_index[r];
        v[i] = make_uint4(0, 0, 0, 0);
        if (r < rows && src >= 0 && c0 + cc < cols) {
          v[i] = *reinterpret_cast<const uint4*>(x + src * ld_x + c0 + cc);
          if (gp.row_scale) {
            const float rs = gp.row_scale[r];
            uint32_t* u = &v[i].x;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float2 t = unpack_bf16(u[j]);
              u[j] = pack_bf16(t.x * rs, t.y * rs);
            }
          }
        }
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4*>(&tile[qtile_at((base + i) * 16 + (tid >> 4), tid & 15)]) = v[i];
    }
  } else {
    // the tile is computed from h (and dout), two rows' loads in flight per thread.
    // GLU_FWD: cols == f, column c pairs h[:, c] with h[:, f + c]. GLU_BWD: cols == 2f and
    // a tile lies in one half (f % 128 == 0): gate gradients, then up gradients.
    const bool up_half = SRC == QSRC_GLU_BWD && c0 >= gp.f;
    const int hc = (up_half ? c0 - gp.f : c0) + cc;  // gate column in h
#pragma unroll 1
    for (int base = 0; base < 8; base += 2) {
      uint4 g[2], u[2], d[2];
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const long r = r0 + (base + i) * 16 + (tid >> 4);
        g[i] = u[i] = d[i] = make_uint4(0, 0, 0, 0);
        if (r < rows && c0 + cc < cols) {
          g[i] = *reinterpret_cast<const uint4*>(x + r * ld_x + hc);
          u[i] = *reinterpret_cast<const uint4*>(x + r * ld_x + gp.f + hc);
          if (SRC == QSRC_GLU_BWD) d[i] = *reinterpret_cast<const uint4*>(gp.dout + r * (long)gp.f + hc);
        }
      }
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const long r = r0 + (base + i) * 16 + (tid >> 4);
        uint4 o = make_uint4(0, 0, 0, 0);
        if (r < rows && c0 + cc < cols)
          o = SRC == QSRC_GLU_FWD ? glu_fwd8(g[i], u[i], gp, gp.row_scale ? gp.row_scale[r] : 1.f)
                                  : glu_bwd8(g[i], u[i], d[i], up_half, gp);
        *reinterpret_cast<uint4*>(&tile[qtile_at((base + i) * 16 + (tid >> 4), tid & 15)]) = o;
      }
    }
  }
  __syncthreads();
  if (q_row) {
    // thread -> row tid % 128, 32-column blocks tid / 128 and tid / 128 + 2
    const int rr = tid & 127;
    const long r = r0 + rr;
#pragma unroll 1
    for (int i = 0; i < 2; ++i) {
      const int cb = (tid >> 7) + 2 * i;
      uint4 w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k) w[k] = *reinterpret_cast<const uint4*>(&tile[qtile_at(rr, cb * 4 + k)]);
      float amax = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint32_t* u = &w[k].x;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 t = unpack_bf16(u[j]);
          amax = fmaxf(amax, fmaxf(fabsf(t.x), fabsf(t.y)));
        }
      }
      const bool live = r < rows && c0 + cb * 32 < cols;
      const uint8_t e = e8m0_of(amax);
      const float inv = e8m0_inv(e);
      sfr[(rr & 31) * 16 + (rr >> 5) * 4 + cb] = live ? e : (uint8_t)127;
      if (live) {
        uint4* dst = reinterpret_cast<uint4*>(q_row + r * cols + c0 + cb * 32);
#pragma unroll
        for (int hv = 0; hv < 2; ++hv) {
          uint32_t packed[4];
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const uint4& ww = w[2 * hv + k];
            const float2 a = unpack_bf16(ww.x), b = unpack_bf16(ww.y), c = unpack_bf16(ww.z), d = unpack_bf16(ww.w);
            packed[2 * k] = cvt_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
            packed[2 * k + 1] = cvt_e4m3x4(c.x * inv, c.y * inv, d.x * inv, d.y * inv);
          }
          dst[hv] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        }
      }
    }
  }
  if (q_col) {
    // A warp takes 8 columns × 32 rows at a time: one transposing ldmatrix hands each thread
    // eight consecutive rows of one column (thread = column t/4, rows 8·(t%4)..+7), the four
    // threads of a column share the block's maximum by two shuffles, and each writes 8 bytes.
    const int warp = tid >> 5, lane = tid & 31;
    const int m = lane >> 3, i = lane & 7;  // this lane addresses row i of matrix m
    const int col = lane >> 2, q = lane & 3;
#pragma unroll 2
    for (int task = 0; task < 8; ++task) {
      const int cg = warp * 2 + (task >> 2), rb = task & 3;
      const int src_row = rb * 32 + 8 * (i >> 1) + 2 * m + (i & 1);
      const uint32_t addr = (uint32_t)__cvta_generic_to_shared(&tile[qtile_at(src_row, cg)]);
      uint32_t w0, w1, w2, w3;
      asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                   : "=r"(w0), "=r"(w1), "=r"(w2), "=r"(w3) : "r"(addr));
      const float2 a = unpack_bf16(w0), b = unpack_bf16(w1), c = unpack_bf16(w2), d = unpack_bf16(w3);
      float amax = fmaxf(fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(b.x), fabsf(b.y))),
                         fmaxf(fmaxf(fabsf(c.x), fabsf(c.y)), fmaxf(fabsf(d.x), fabsf(d.y))));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      const int ccol = cg * 8 + col;
      const bool live = c0 + ccol < cols;
      const uint8_t e = e8m0_of(amax);
      const float inv = e8m0_inv(e);
      if (q == 0) sfc[(ccol & 31) * 16 + (ccol >> 5) * 4 + rb] = live ? e : (uint8_t)127;
      if (live) {
        uint2 out;
        out.x = cvt_e4m3x4(a.x * inv, a.y * inv, b.x * inv, b.y * inv);
        out.y = cvt_e4m3x4(c.x * inv, c.y * inv, d.x * inv, d.y * inv);
        *reinterpret_cast<uint2*>(q_col + (size_t)(c0 + ccol) * ld_col + r0 + rb * 32 + 8 * q) = out;
      }
    }
  }
  __syncthreads();
  // one whole 512-byte scale tile per output
  if (q_row && tid < 32) {
    uint8_t* dst = sf_row + ((size_t)blockIdx.y * (sf_cols_row >> 2) + blockIdx.x) * 512;
    reinterpret_cast<uint4*>(dst)[tid] = reinterpret_cast<const uint4*>(sfr)[tid];
  }
  if (q_col && tid >= 32 && tid < 64) {
    uint8_t* dst = sf_col + ((size_t)blockIdx.x * (sf_cols_col >> 2) + blockIdx.y) * 512;
    reinterpret_cast<uint4*>(dst)[tid - 32] = reinterpret_cast<const uint4*>(sfc)[tid - 32];
  }
}

// ---------------------------------------------------------------- NVFP4 quantiser
// x [rows, cols] bf16 -> E2M1 codes, two per byte (low nibble first), in blocks of 16 along a
// row with one E4M3 scale each, under one fp32 scale for the tensor (*tensor_scale =
// amax / (6 * 448), taken by the caller's reduction). One thread per block: two 16-byte loads,
// the block's largest magnitude, its scale rounded to E4M3, sixteen values rounded to nearest
// by the hardware's E2M1 conversion, one 8-byte store.
__global__ void quant_nvfp4_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ tensor_scale,
                                   uint8_t* __restrict__ packed, uint8_t* __restrict__ scales, long blocks) {
  const float ts = *tensor_scale;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < blocks; i += (long)gridDim.x * blockDim.x) {
    const uint4 a = *reinterpret_cast<const uint4*>(x + i * 16);
    const uint4 b = *reinterpret_cast<const uint4*>(x + i * 16 + 8);
    float v[16];
    const uint32_t* au = &a.x; const uint32_t* bu = &b.x;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 f = unpack_bf16(au[q]), g = unpack_bf16(bu[q]);
      v[2 * q] = f.x; v[2 * q + 1] = f.y; v[8 + 2 * q] = g.x; v[8 + 2 * q + 1] = g.y;
    }
    float amax = 0.f;
#pragma unroll
    for (int q = 0; q < 16; ++q) amax = fmaxf(amax, fabsf(v[q]));
    const __nv_fp8_storage_t sbyte = __nv_cvt_float_to_fp8(fminf(__fdiv_rn(amax, 6.f * ts), 448.f), __NV_SATFINITE, __NV_E4M3);
    const float scale = __half2float(__half(__nv_cvt_fp8_to_halfraw(sbyte, __NV_E4M3)));
    const float denom = scale * ts;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float lo = denom > 0.f ? __fdiv_rn(v[2 * q], denom) : 0.f;
      const float hi = denom > 0.f ? __fdiv_rn(v[2 * q + 1], denom) : 0.f;
      const uint32_t byte = (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
      w[q >> 2] |= (byte & 0xffu) << (8 * (q & 3));
    }
    *reinterpret_cast<uint2*>(packed + i * 8) = make_uint2(w[0], w[1]);
    scales[i] = sbyte;
  }
}

// ---------------------------------------------------------------- cross-entropy
// One block per row of a logits chunk [rows, vocab] (bf16). Writes per-row loss and
// logZ (fp32) and overwrites the logits with dlogits = (softmax - onehot) * grad_scale
// * mask (+ z-loss term), ready for the dX / dW GEMMs.
__global__ void ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const int* __restrict__ targets,
                                  const float* __restrict__ mask, float* __restrict__ loss,
                                  float* __restrict__ logz_out, int vocab, long ld, float grad_scale,
                                  float z_weight, float softcap) {
  const long row = blockIdx.x;
  __nv_bfloat16* lr = logits + row * ld;
  __shared__ float red[32];
  __shared__ float bcast[2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  float mx = -INFINITY;
  for (int i = threadIdx.x * 8; i < vocab; i += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(lr + i);
    const uint32_t* u = &v.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = unpack_bf16(u[j]);
      if (softcap > 0.f) { t.x = softcap * tanhf(t.x / softcap); t.y = softcap * tanhf(t.y / softcap); }
      mx = fmaxf(mx, fmaxf(t.x, t.y));
    }
  }
  mx = warp_max(mx);
  if (lane == 0) red[warp] = mx;
  __syncthreads();
  if (warp == 0) { float v = lane < nw ? red[lane] : -INFINITY; v = warp_max(v); if (lane == 0) bcast[0] = v; }
  __syncthreads();
  mx = bcast[0];
  float sum = 0.f;
  for (int i = threadIdx.x * 8; i < vocab; i += blockDim.x * 8) {
    const uint4 v = *reinterpret_cast<const uint4*>(lr + i);
    const uint32_t* u = &v.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = unpack_bf16(u[j]);
      if (softcap > 0.f) { t.x = softcap * tanhf(t.x / softcap); t.y = softcap * tanhf(t.y / softcap); }
      sum += __expf(t.x - mx) + __expf(t.y - mx);
    }
  }
  sum = warp_sum(sum);
  __syncthreads();
  if (lane == 0) red[warp] = sum;
  __syncthreads();
  if (warp == 0) { float v = lane < nw ? red[lane] : 0.f; v = warp_sum(v); if (lane == 0) bcast[1] = v; }
  __syncthreads();
  sum = bcast[1];
  const float logz = mx + logf(sum);
  const int tgt = targets[row];
  const float m = mask ? mask[row] : 1.f;
  if (threadIdx.x == 0) {
    float t = __bfloat162float(lr[tgt]);
    if (softcap > 0.f) t = softcap * tanhf(t / softcap);
    loss[row] = (logz - t + z_weight * logz * logz) * m;
    if (logz_out) logz_out[row] = logz;
  }
  __syncthreads();  // the target logit is read before it is overwritten below
  const float gs = grad_scale * m;
  const float zfac = 1.f + 2.f * z_weight * logz;
  const float inv = 1.f / sum;
  for (int i = threadIdx.x * 8; i < vocab; i += blockDim.x * 8) {
    uint4 v = *reinterpret_cast<const uint4*>(lr + i);
    uint32_t* u = &v.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 t = unpack_bf16(u[j]);
      float dcap0 = 1.f, dcap1 = 1.f;
      if (softcap > 0.f) {
        const float a = tanhf(t.x / softcap), b = tanhf(t.y / softcap);
        t.x = softcap * a; t.y = softcap * b; dcap0 = 1.f - a * a; dcap1 = 1.f - b * b;
      }
      float p0 = __expf(t.x - mx) * inv * zfac, p1 = __expf(t.y - mx) * inv * zfac;
      if (i + 2 * j == tgt) p0 -= 1.f;
      if (i + 2 * j + 1 == tgt) p1 -= 1.f;
      u[j] = pack_bf16(p0 * gs * dcap0, p1 * gs * dcap1);
    }
    *reinterpret_cast<uint4*>(lr + i) = v;
  }
}

// ---------------------------------------------------------------- AdamW over flat buffers
// p: fp32 master (or bf16 master when MASTER_BF16), g: bf16 or fp32 grads, optional
// bf16 shadow copy of the updated weights. Moments: fp32, bf16, or 8-bit block-scaled
// (e4m3 values with one E8M0 scale per 32 elements; the second moment is stored as its
// square root so that its dynamic range fits).
// Each lane owns 8 consecutive elements (one 128-bit access of bf16); four adjacent
// lanes form one 32-element scale block of the 8-bit moments and share its amax by
// two shuffles. The buffer length may be ragged: tail elements take scalar paths.
template <typename TT> struct Vec8;
template <> struct Vec8<float> {
  static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  }
  static __device__ __forceinline__ void store(float* p, const float (&f)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
  }
};
template <> struct Vec8<__nv_bfloat16> {
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    float2 t;
    t = unpack_bf16(v.x); f[0] = t.x; f[1] = t.y;
    t = unpack_bf16(v.y); f[2] = t.x; f[3] = t.y;
    t = unpack_bf16(v.z); f[4] = t.x; f[5] = t.y;
    t = unpack_bf16(v.w); f[6] = t.x; f[7] = t.y;
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&f)[8]) {
    uint4 v;
    v.x = pack_bf16(f[0], f[1]); v.y = pack_bf16(f[2], f[3]);
    v.z = pack_bf16(f[4], f[5]); v.w = pack_bf16(f[6], f[7]);
    *reinterpret_cast<uint4*>(p) = v;
  }
};

template <typename PT, typename GT, int MOM>
__global__ void adamw_kernel(PT* __restrict__ p, const GT* __restrict__ g, void* __restrict__ m_,
                             void* __restrict__ v_, uint8_t* __restrict__ m_sf, uint8_t* __restrict__ v_sf,
                             __nv_bfloat16* __restrict__ shadow, long n, float lr, float b1, float b2,
                             float eps, float wd, float bc1, float bc2, const float* __restrict__ grad_scale_ptr,
                             float grad_scale_const) {
  const float gscale = grad_scale_ptr ? *grad_scale_ptr * grad_scale_const : grad_scale_const;
  const long groups = (n + 7) / 8;
  // whole warps iterate together so that the 4-lane shuffles below are always converged
  const long warp_groups = (groups + 31) / 32 * 32;
  for (long gi = (long)blockIdx.x * blockDim.x + threadIdx.x; gi < warp_groups; gi += (long)gridDim.x * blockDim.x) {
    const long i0 = gi * 8;
    const bool active = i0 < n;
    const bool full = i0 + 8 <= n;
    const int cnt = active ? (int)min(8L, n - i0) : 0;
    float pw[8], gr[8], pm[8], pv[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) { pw[j] = 0.f; gr[j] = 0.f; pm[j] = 0.f; pv[j] = 0.f; }
    if (full) {
      Vec8<PT>::load(p + i0, pw);
      Vec8<GT>::load(g + i0, gr);
    } else {
      _Pragma("unroll") for (int j = 0; j < 8; ++j) if (j < cnt) { pw[j] = (float)p[i0 + j]; gr[j] = (float)g[i0 + j]; }
    }
    const long blk = i0 >> 5;
    if (MOM == MOM_F32) {
      if (full) { Vec8<float>::load(reinterpret_cast<float*>(m_) + i0, pm); Vec8<float>::load(reinterpret_cast<float*>(v_) + i0, pv); }
      else _Pragma("unroll") for (int j = 0; j < 8; ++j) if (j < cnt) { pm[j] = reinterpret_cast<float*>(m_)[i0 + j]; pv[j] = reinterpret_cast<float*>(v_)[i0 + j]; }
    } else if (MOM == MOM_BF16) {
      if (full) { Vec8<__nv_bfloat16>::load(reinterpret_cast<__nv_bfloat16*>(m_) + i0, pm); Vec8<__nv_bfloat16>::load(reinterpret_cast<__nv_bfloat16*>(v_) + i0, pv); }
      else _Pragma("unroll") for (int j = 0; j < 8; ++j) if (j < cnt) {
        pm[j] = __bfloat162float(reinterpret_cast<__nv_bfloat16*>(m_)[i0 + j]);
        pv[j] = __bfloat162float(reinterpret_cast<__nv_bfloat16*>(v_)[i0 + j]);
      }
    } else if (active) {
      const float sm = __uint_as_float((uint32_t)max((int)m_sf[blk], 1) << 23);
      const float sv = __uint_as_float((uint32_t)max((int)v_sf[blk], 1) << 23);
      // the eight moment bytes of m and of v travel as two 32-bit words each (no byte arrays:
      // those would live in local memory)
      uint2 mw = make_uint2(0, 0), vw = make_uint2(0, 0);
      if (full) {
        mw = *reinterpret_cast<const uint2*>(reinterpret_cast<uint8_t*>(m_) + i0);
        vw = *reinterpret_cast<const uint2*>(reinterpret_cast<uint8_t*>(v_) + i0);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          if (j < cnt) {
            const uint32_t bm = reinterpret_cast<uint8_t*>(m_)[i0 + j], bv = reinterpret_cast<uint8_t*>(v_)[i0 + j];
            if (j < 4) { mw.x |= bm << (8 * j); vw.x |= bv << (8 * j); }
            else { mw.y |= bm << (8 * (j - 4)); vw.y |= bv << (8 * (j - 4)); }
          }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {  // two values per conversion
        const __nv_fp8x2_storage_t m2 = (__nv_fp8x2_storage_t)(((j < 2 ? mw.x : mw.y) >> (16 * (j & 1))) & 0xffffu);
        const __nv_fp8x2_storage_t v2 = (__nv_fp8x2_storage_t)(((j < 2 ? vw.x : vw.y) >> (16 * (j & 1))) & 0xffffu);
        const float2 fm = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(m2, __NV_E4M3)));
        const float2 fv = __half22float2(__half2(__nv_cvt_fp8x2_to_halfraw2(v2, __NV_E4M3)));
        pm[2 * j] = fm.x * sm; pm[2 * j + 1] = fm.y * sm;
        const float r0 = fv.x * sv, r1 = fv.y * sv;
        pv[2 * j] = r0 * r0; pv[2 * j + 1] = r1 * r1;
      }
    }
    // one approximate square root and one approximate reciprocal per element (the special
    // function unit): the exact forms cost more instructions than the memory traffic hides
    float am = 0.f, av = 0.f;
    float sq[8];
    const float ibc1 = 1.f / bc1, isb2 = rsqrtf(bc2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gg = gr[j] * gscale;
      pm[j] = b1 * pm[j] + (1.f - b1) * gg;
      pv[j] = b2 * pv[j] + (1.f - b2) * gg * gg;
      asm("sqrt.approx.f32 %0, %1;" : "=f"(sq[j]) : "f"(pv[j]));
      const float upd = __fdividef(pm[j] * ibc1, fmaf(sq[j], isb2, eps)) + wd * pw[j];
      pw[j] -= lr * upd;
      if (j < cnt) { am = fmaxf(am, fabsf(pm[j])); av = fmaxf(av, sq[j]); }
    }
    if (full) {
      Vec8<PT>::store(p + i0, pw);
      if (shadow) Vec8<__nv_bfloat16>::store(shadow + i0, pw);
    } else {
      _Pragma("unroll") for (int j = 0; j < 8; ++j) if (j < cnt) { p[i0 + j] = (PT)pw[j]; if (shadow) shadow[i0 + j] = __float2bfloat16(pw[j]); }
    }
    if (MOM == MOM_F32) {
      if (full) { Vec8<float>::store(reinterpret_cast<float*>(m_) + i0, pm); Vec8<float>::store(reinterpret_cast<float*>(v_) + i0, pv); }
      else _Pragma("unroll") for (int j = 0; j < 8; ++j) if (j < cnt) { reinterpret_cast<float*>(m_)[i0 + j] = pm[j]; reinterpret_cast<float*>(v_)[i0 + j] = pv[j]; }
    } else if (MOM == MOM_BF16) {
      if (full) { Vec8<__nv_bfloat16>::store(reinterpret_cast<__nv_bfloat16*>(m_) + i0, pm); Vec8<__nv_bfloat16>::store(reinterpret_cast<__nv_bfloat16*>(v_) + i0, pv); }
      else _Pragma("unroll") for (int j = 0; j < 8; ++j) if (j < cnt) {
        reinterpret_cast<__nv_bfloat16*>(m_)[i0 + j] = __float2bfloat16(pm[j]);
        reinterpret_cast<__nv_bfloat16*>(v_)[i0 + j] = __float2bfloat16(pv[j]);
      }
    } else {
      // amax over the 4 lanes of the scale block
      am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 1)); am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, 2));
      av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 1)); av = fmaxf(av, __shfl_xor_sync(0xffffffffu, av, 2));
      if (active) {
        const uint8_t em = (uint8_t)max((int)e8m0_of(am), 1), ev = (uint8_t)max((int)e8m0_of(av), 1);
        const float im = e8m0_inv(em), iv = e8m0_inv(ev);
        if ((threadIdx.x & 3) == 0) { m_sf[blk] = em; v_sf[blk] = ev; }
        uint2 mo = make_uint2(0, 0), vo = make_uint2(0, 0);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t m2 = __nv_cvt_float2_to_fp8x2(make_float2(pm[2 * j] * im, pm[2 * j + 1] * im), __NV_SATFINITE, __NV_E4M3);
          const uint32_t v2 = __nv_cvt_float2_to_fp8x2(make_float2(sq[2 * j] * iv, sq[2 * j + 1] * iv), __NV_SATFINITE, __NV_E4M3);
          if (j < 2) { mo.x |= m2 << (16 * j); vo.x |= v2 << (16 * j); }
          else { mo.y |= m2 << (16 * (j - 2)); vo.y |= v2 << (16 * (j - 2)); }
        }
        if (full) {
          *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(m_) + i0) = mo;
          *reinterpret_cast<uint2*>(reinterpret_cast<uint8_t*>(v_) + i0) = vo;
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (j < cnt) {
              reinterpret_cast<uint8_t*>(m_)[i0 + j] = (uint8_t)(((j < 4 ? mo.x : mo.y) >> (8 * (j & 3))) & 0xff);
              reinterpret_cast<uint8_t*>(v_)[i0 + j] = (uint8_t)(((j < 4 ? vo.x : vo.y) >> (8 * (j & 3))) & 0xff);
            }
        }
      }
    }
  }
}

// sum of squares of a flat buffer into out[0] (fp32 atomics), for the global grad norm
template <typename GT>
__global__ void sumsq_kernel(const GT* __restrict__ g, long n, float* __restrict__ out) {
  float s = 0.f;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float v = (float)g[i];
    s += v * v;
  }
  s = warp_sum(s);
  __shared__ float red[32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = s;
  __syncthreads();
  if (warp == 0) {
    float v = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    v = warp_sum(v);
    if (lane == 0) atomicAdd(out, v);
  }
}

// ---------------------------------------------------------------- router top-k
// The k largest of each row of scores [rows, n] (fp32), indices in descending order of value
// (ties: the lower index first). One warp per row; lane l holds columns l, l + 32, ... in
// registers and the warp picks one winner per round by shuffles.
template <int NV>
__global__ void topk_rows_kernel(const float* __restrict__ scores, long* __restrict__ idx, long rows, int n, int k) {
  const int lane = threadIdx.x & 31;
  const long row = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* sr = scores + row * n;
  float v[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int c = j * 32 + lane;
    v[j] = c < n ? sr[c] : -INFINITY;
    if (v[j] != v[j]) v[j] = -INFINITY;  // a NaN never wins
  }
  for (int round = 0; round < k; ++round) {
    float best = -INFINITY;
    int at = 0x7fffffff;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      const int c = j * 32 + lane;
      if (c < n && (v[j] > best || (v[j] == best && c < at))) { best = v[j]; at = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (lane == 0) idx[row * k + round] = at;
#pragma unroll
    for (int j = 0; j < NV; ++j)
      if (j * 32 + lane == at) v[j] = -INFINITY;  // taken: out of the next rounds
  }
}

// ---------------------------------------------------------------- MoE gather / combine
// out[r] = x[index[r]] (zero row when index[r] < 0); rows of d bf16, d % 8 == 0.
__global__ void gather_rows_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ index,
                                   __nv_bfloat16* __restrict__ out, long rows, int d) {
  const int vec = d / 8;
  const long total = rows * vec;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / vec; const int c = (int)(i % vec);
    const int src = index[r];
    uint4 v = make_uint4(0, 0, 0, 0);
    if (src >= 0) v = reinterpret_cast<const uint4*>(x + (long)src * d)[c];
    reinterpret_cast<uint4*>(out + r * d)[c] = v;
  }
}
// out[t] = sum_k w[t,k] * y[pos[t,k]]  (pos < 0 = dropped pick); w may be null (= 1).
__global__ void combine_rows_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ pos,
                                    const float* __restrict__ w, __nv_bfloat16* __restrict__ out,
                                    long tokens, int k, int d) {
  const int vec = d / 8;
  const long total = tokens * vec;
  for (long i = (long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long t = i / vec; const int c = (int)(i % vec);
    float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int j = 0; j < k; ++j) {
      const int r = pos[t * k + j];
      if (r < 0) continue;
      const float ww = w ? w[t * k + j] : 1.f;
      const uint4 v = reinterpret_cast<const uint4*>(y + (long)r * d)[c];
      const uint32_t* u = &v.x;
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = unpack_bf16(u[q]); acc[2 * q] += ww * f.x; acc[2 * q + 1] += ww * f.y; }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + t * d)[c] = o;
  }
}

// Backward of the weighted combine, one warp per pick (t, j) with r = pos[t,j]:
//   dy[r] = w[t,j] * dout[t]     dw[t,j] = <y[r], dout[t]>     (dropped picks: dw = 0)
__global__ void combine_bwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ dout,
                                   const int* __restrict__ pos, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ dy, float* __restrict__ dw,
                                   long picks, int k, int d) {
  const int lane = threadIdx.x & 31;
  const int vec = d / 8;
  for (long i = (long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); i < picks;
       i += (long)gridDim.x * (blockDim.x >> 5)) {
    const int r = pos[i];
    if (r < 0) { if (lane == 0 && dw) dw[i] = 0.f; continue; }
    const long t = i / k;
    const float ww = w ? w[i] : 1.f;
    float dot = 0.f;
    for (int c = lane; c < vec; c += 32) {
      const uint4 g = reinterpret_cast<const uint4*>(dout + t * d)[c];
      const uint32_t* gu = &g.x;
      uint4 o; uint32_t* ou = &o.x;
      uint4 yv = make_uint4(0, 0, 0, 0);
      if (dw) yv = reinterpret_cast<const uint4*>(y + (long)r * d)[c];
      const uint32_t* yu = &yv.x;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 gf = unpack_bf16(gu[q]);
        const float2 yf = unpack_bf16(yu[q]);
        dot += gf.x * yf.x + gf.y * yf.y;
        ou[q] = pack_bf16(gf.x * ww, gf.y * ww);
      }
      if (dy) reinterpret_cast<uint4*>(dy + (long)r * d)[c] = o;
    }
    if (dw) {
      dot = warp_sum(dot);
      if (lane == 0) dw[i] = dot;
    }
  }
}

// ---------------------------------------------------------------- launchers
static inline int grid_for(long work, int per_block, int cap = 148 * 16) {
  long g = (work + per_block - 1) / per_block;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

void rmsnorm_fwd(const void* x, const float* w, void* y, float* rstd, long rows, int d, float eps, cudaStream_t s) {
  const int wpb = 8;
  rmsnorm_fwd_kernel<8><<<(int)((rows + wpb - 1) / wpb), wpb * 32, 0, s>>>(
      (const __nv_bfloat16*)x, w, (__nv_bfloat16*)y, rstd, (int)rows, d, eps);
}
void rmsnorm_bwd(const void* x, const float* w, const void* dy, const float* rstd, void* dx, float* dw, long rows, int d, cudaStream_t s) {
  const int wpb = 8;
  int grid = (int)min((rows + wpb - 1) / wpb, 148L * 4);
  const size_t slab_bytes = (size_t)wpb * d * sizeof(float);
  if (d % 8 == 0 && slab_bytes <= 200 * 1024) {
    if (slab_bytes > 48 * 1024)  // per device, so set at every launch that needs it (a cheap call)
      cudaFuncSetAttribute(rmsnorm_bwd_slab_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)slab_bytes);
    rmsnorm_bwd_slab_kernel<<<grid, wpb * 32, slab_bytes, s>>>((const __nv_bfloat16*)x, w, (const __nv_bfloat16*)dy, rstd, (__nv_bfloat16*)dx, dw, (int)rows, d);
    return;
  }
  rmsnorm_bwd_kernel<<<grid, wpb * 32, d * sizeof(float), s>>>(
      (const __nv_bfloat16*)x, w, (const __nv_bfloat16*)dy, rstd, (__nv_bfloat16*)dx, dw, (int)rows, d);
}
const char* norm_rope(bool bwd, const void* x, const float* w, const float* cs, const float* sn, void* y,
                      float* rstd, const void* dy, float* dw, long tokens, int heads, int D,
                      long stride_x, long stride_y, float eps, cudaStream_t s) {
  const int wpb = 8;
  const long items = (tokens * heads + (256 / D) - 1) / (256 / D);  // warp steps: 256 / D items each
  int grid = (int)min((items + wpb - 1) / wpb, 148L * 8);
#define NR_CASE(D_) \
  if (D == D_) { \
    if (bwd) norm_rope_kernel<D_, true><<<grid, wpb * 32, 0, s>>>((const __nv_bfloat16*)x, w, cs, sn, (__nv_bfloat16*)y, rstd, (const __nv_bfloat16*)dy, dw, tokens, heads, stride_x, stride_y, eps); \
    else     norm_rope_kernel<D_, false><<<grid, wpb * 32, 0, s>>>((const __nv_bfloat16*)x, w, cs, sn, (__nv_bfloat16*)y, rstd, nullptr, nullptr, tokens, heads, stride_x, stride_y, eps); \
    return nullptr; }
  NR_CASE(64) NR_CASE(128) NR_CASE(256)
#undef NR_CASE
  return "norm_rope: head_dim must be 64, 128 or 256";
}
void glu_fwd(const void* h, void* out, const float* row_scale, long rows, int f, int kind, float limit, float up_offset, cudaStream_t s) {
  glu_fwd_kernel<<<grid_for(rows * (f / 8), 256), 256, 0, s>>>((const __nv_bfloat16*)h, (__nv_bfloat16*)out, row_scale, rows, f, kind, limit, up_offset);
}
void glu_bwd(const void* h, const void* dout, void* dh, const float* row_scale, float* d_row_scale, long rows, int f, int kind, float limit, float up_offset, cudaStream_t s) {
  glu_bwd_kernel<<<grid_for(rows * (f / 8), 256), 256, 0, s>>>((const __nv_bfloat16*)h, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dh, row_scale, d_row_scale, rows, f, kind, limit, up_offset);
}
void quant_mxfp8(const void* x, long ld_x, const int* row_index, const float* row_scale, uint8_t* q_row, uint8_t* sf_row, uint8_t* q_col, uint8_t* sf_col, long rows, int cols, long ld_col, int batch, long x_batch_stride, cudaStream_t s) {
  const long extent = q_col ? (ld_col > rows ? ld_col : rows) : rows;  // the transposed copy is padded to ld_col
  dim3 grid((cols + 127) / 128, (unsigned)((extent + 127) / 128), batch);
  quant_mxfp8_kernel<QSRC_PLAIN><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, ld_x, row_index, q_row, sf_row, q_col, sf_col, rows, cols, ld_col, x_batch_stride, QuantGlu{row_scale, nullptr, 0, 0, 0.f, 0.f, nullptr});
}
void requant_mxfp8_cols(const uint8_t* q, const uint8_t* sf, uint8_t* q_col, uint8_t* sf_col, long rows, int cols,
                        long ld_col, cudaStream_t s) {
  const long extent = ld_col > rows ? ld_col : rows;
  dim3 grid((cols + 127) / 128, (unsigned)((extent + 127) / 128), 1);
  quant_mxfp8_kernel<QSRC_MX><<<grid, 256, 0, s>>>((const __nv_bfloat16*)q, cols, nullptr, nullptr, nullptr, q_col, sf_col,
                                                   rows, cols, ld_col, 0, QuantGlu{nullptr, nullptr, 0, 0, 0.f, 0.f, sf});
}
void quant_mxfp8_glu(const void* h, const void* dout, const float* row_scale, uint8_t* q_row, uint8_t* sf_row,
                     uint8_t* q_col, uint8_t* sf_col, long rows, int f, long ld_col, int kind, float limit,
                     float up_offset, cudaStream_t s) {
  const int cols = dout ? 2 * f : f;
  const long extent = q_col ? (ld_col > rows ? ld_col : rows) : rows;
  dim3 grid((cols + 127) / 128, (unsigned)((extent + 127) / 128), 1);
  QuantGlu gp{dout ? nullptr : row_scale, (const __nv_bfloat16*)dout, f, kind, limit, up_offset, nullptr};
  if (dout) quant_mxfp8_kernel<QSRC_GLU_BWD><<<grid, 256, 0, s>>>((const __nv_bfloat16*)h, 2L * f, nullptr, q_row, sf_row, q_col, sf_col, rows, cols, ld_col, 0, gp);
  else quant_mxfp8_kernel<QSRC_GLU_FWD><<<grid, 256, 0, s>>>((const __nv_bfloat16*)h, 2L * f, nullptr, q_row, sf_row, q_col, sf_col, rows, cols, ld_col, 0, gp);
}
void quant_nvfp4(const void* x, const float* tensor_scale, uint8_t* packed, uint8_t* scales, long rows, int cols,
                 cudaStream_t s) {
  const long blocks = rows * (cols / 16);
  quant_nvfp4_kernel<<<grid_for(blocks, 256), 256, 0, s>>>((const __nv_bfloat16*)x, tensor_scale, packed, scales, blocks);
}
void ce_fwd_bwd(void* logits, const int* targets, const float* mask, float* loss, float* logz, long rows, int vocab, long ld, float grad_scale, float z_weight, float softcap, cudaStream_t s) {
  ce_fwd_bwd_kernel<<<(unsigned)rows, 512, 0, s>>>((__nv_bfloat16*)logits, targets, mask, loss, logz, vocab, ld, grad_scale, z_weight, softcap);
}
const char* adamw(void* p, bool p_bf16, const void* g, bool g_bf16, void* m, void* v, uint8_t* m_sf, uint8_t* v_sf, int mom,
                  void* shadow, long n, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2,
                  const float* gscale_ptr, float gscale, cudaStream_t s) {
  const int grid = grid_for((n + 7) / 8, 256, 148 * 32);
#define AW(PT, GT, MOM_) adamw_kernel<PT, GT, MOM_><<<grid, 256, 0, s>>>((PT*)p, (const GT*)g, m, v, m_sf, v_sf, (__nv_bfloat16*)shadow, n, lr, b1, b2, eps, wd, bc1, bc2, gscale_ptr, gscale)
#define AW_MOM(PT, GT) { if (mom == MOM_F32) AW(PT, GT, MOM_F32); else if (mom == MOM_BF16) AW(PT, GT, MOM_BF16); else AW(PT, GT, MOM_FP8); return nullptr; }
  if (!p_bf16 && g_bf16) AW_MOM(float, __nv_bfloat16)
  if (!p_bf16 && !g_bf16) AW_MOM(float, float)
  if (p_bf16 && g_bf16) AW_MOM(__nv_bfloat16, __nv_bfloat16)
  if (p_bf16 && !g_bf16) AW_MOM(__nv_bfloat16, float)
#undef AW_MOM
#undef AW
  return "adamw: unsupported dtypes";
}
void sumsq(const void* g, bool bf16, long n, float* out, cudaStream_t s) {
  const int grid = grid_for(n, 256 * 8, 148 * 8);
  if (bf16) sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)g, n, out);
  else sumsq_kernel<float><<<grid, 256, 0, s>>>((const float*)g, n, out);
}
const char* topk_rows(const float* scores, long* idx, long rows, int n, int k, cudaStream_t s) {
  const int wpb = 8;
  const unsigned grid = (unsigned)((rows + wpb - 1) / wpb);
#define TK_CASE(NV_) if (n <= NV_ * 32) { topk_rows_kernel<NV_><<<grid, wpb * 32, 0, s>>>(scores, idx, rows, n, k); return nullptr; }
  TK_CASE(1) TK_CASE(2) TK_CASE(4) TK_CASE(8) TK_CASE(16)
#undef TK_CASE
  return "topk_rows: at most 512 columns";
}
void gather_rows(const void* x, const int* index, void* out, long rows, int d, cudaStream_t s) {
  gather_rows_kernel<<<grid_for(rows * (d / 8), 256), 256, 0, s>>>((const __nv_bfloat16*)x, index, (__nv_bfloat16*)out, rows, d);
}
void combine_bwd(const void* y, const void* dout, const int* pos, const float* w, void* dy, float* dw, long picks, int k, int d, cudaStream_t s) {
  combine_bwd_kernel<<<grid_for(picks, 8), 256, 0, s>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)dout, pos, w, (__nv_bfloat16*)dy, dw, picks, k, d);
}
void combine_rows(const void* y, const int* pos, const float* w, void* out, long tokens, int k, int d, cudaStream_t s) {
  combine_rows_kernel<<<grid_for(tokens * (d / 8), 256), 256, 0, s>>>((const __nv_bfloat16*)y, pos, w, (__nv_bfloat16*)out, tokens, k, d);
}

}  // namespace bux
