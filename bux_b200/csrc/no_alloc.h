// A C entry point for callers that cannot allocate device memory.
//
// This has no counterpart in the reference framework. It exists for hosts that embed
// this library where cudaMalloc is off limits: plugins that must stay within a memory
// budget fixed at start-up, processes whose device allocator belongs to someone else (an
// inference server's arena that hands out the whole GPU), and latency-bound loops that
// cannot afford a driver allocation (it synchronises the device). Such a caller
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

// The kernels' waits (on their own barriers) are bounded; one that runs out makes the
// kernel return early and records where in a status word that also lives inside the
// library, so a call that returned 0 may still have produced no dk/dv. This reads that
// word on the current device after the work queued so far has finished (it blocks):
// *code is 0 when no wait ran out, else kernel << 24 | site << 16 | block; *count is the
// number of waits that ran out since the word was last cleared. `clear` != 0 resets it.
// Returns 0, or 3 / 4 as above. Either pointer may be null.
int bux_attn_bwd_static_status(unsigned int* code, unsigned int* count, int clear);

#ifdef __cplusplus
}
#endif
