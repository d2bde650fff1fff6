// A C entry point for callers that cannot allocate device memory.
//
// This has no counterpart in the reference framework. It exists for hosts that embed
// this library where cudaMalloc is off limits: inside a CUDA-graph capture or another
// framework's stream-ordered region where an allocation would break the capture, in
// plugins that must stay within a memory budget fixed at start-up, or in processes
// whose allocator belongs to someone else (an inference server's arena). Such a caller
// owns every input and output buffer and hands over raw device pointers; the one
// piece of memory the attention backward needs beyond those (its per-row
// sum(dO * O) table) lives in a fixed array inside the library.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// Largest batch * query_heads * query_length the built-in scratch holds (floats).
#define BUX_ATTN_BWD_STATIC_MAX_ROWS (1 << 22)

// Softmax-attention backward with no allocation of any kind.
//   q, o, d_o: [B, T, H, D] bf16      k, v: [B, S, G, D] bf16      lse: [B, H, T] fp32
//   dq: [B, T, H, D] fp32 (cleared here, then accumulated)   dk, dv: [B, S, G, D] bf16
//   sinks, dsinks: [H] fp32 or null (dsinks is cleared here)  D is 64 or 128.
// Returns 0 on success; 1 if B*H*T exceeds BUX_ATTN_BWD_STATIC_MAX_ROWS; 2 for an
// unsupported shape; 3 if the scratch address could not be resolved on this device;
// 4 if a launch failed. `message`, when not null, receives a static description.
//
// The first call on each device resolves the scratch array's device address (a
// synchronous driver query): make that first call outside any stream capture. Every
// call on a device shares the one scratch array, so two calls whose kernels can overlap
// on the GPU (different streams, no ordering between them) race on it; order them.
int bux_attn_bwd_static(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                        const float* lse, float* dq, void* dk, void* dv, const float* sinks,
                        float* dsinks, int B, int T, int S, int H, int G, int D, float scale,
                        int causal, int window, void* cuda_stream, const char** message);

#ifdef __cplusplus
}
#endif
