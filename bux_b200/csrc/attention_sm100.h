// Host-visible types of the tcgen05 attention kernels (attention_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bux {

struct Status;

// q, o, d_o, dq: [B, T, H, D] bf16.  k, v, dk, dv: [B, S, G, D] bf16 (H % G == 0).
// lse, delta: [B, H, T] fp32.  sinks / dsinks: [H] fp32 or null.  D is 64 or 128.
// Causal alignment is bottom-right (query t sees keys <= t + S - T); window > 0 keeps
// keys in (t + S - T - window, t + S - T].
// Documents packed into a row (self-attention, T == S): row_lo[b, t] is the first key that
// query t may see (the start of its document) and key_hi[b, s] the last query that may see
// key s (the end of its document); both int32, both non-decreasing along a row, or null.
// The forward and the mask use row_lo; key_hi only bounds the backward's walk over query tiles.
struct AttnArgs {
  const void* q = nullptr; const void* k = nullptr; const void* v = nullptr;
  void* o = nullptr; float* lse = nullptr;
  const void* d_o = nullptr; void* dq = nullptr; void* dk = nullptr; void* dv = nullptr;
  float* delta = nullptr;
  const float* sinks = nullptr; float* dsinks = nullptr;
  const int* row_lo = nullptr; const int* key_hi = nullptr;
  int B = 0, T = 0, S = 0, H = 0, G = 0, D = 0;
  float scale = 1.f; bool causal = true; int window = 0;
  Status* status = nullptr;
  // backward only, optional: 32 counters that the CTA of the first key tile adds the cycles of
  // its phases to (softmax warp 0: slots 0-13, MMA issuer: 16-23), for reading the schedule
  unsigned int* phase_cycles = nullptr;
};

const char* attn_fwd_launch(const AttnArgs& a, cudaStream_t stream);
const char* attn_bwd_launch(const AttnArgs& a, cudaStream_t stream);

}  // namespace bux
