// Implementation of the allocation-free attention backward (see no_alloc.h).
#include "no_alloc.h"

#include <cuda_runtime.h>

#include "attention_sm100.h"
#include "common.cuh"

namespace {

// The backward's only scratch: delta[b, h, t] = sum_d dO * O. 16 MiB per GPU that loads
// the library, held until the process exits. Fully rewritten by every call for the rows
// that call uses, so nothing needs clearing between calls.
static __device__ __align__(256) float g_delta_scratch[BUX_ATTN_BWD_STATIC_MAX_ROWS];
// Where the kernels' bounded waits report (see common.cuh).
static __device__ __align__(256) bux::Status g_status_scratch;

constexpr int kMaxDevices = 64;
float* g_delta_ptr[kMaxDevices] = {};
bux::Status* g_status_ptr[kMaxDevices] = {};

// In host code `g_delta_scratch` is only a handle for the symbol; the address a kernel
// can use has to be asked for, once per device, with that device current.
bool resolve(int device) {
  if (g_delta_ptr[device] != nullptr) return true;
  void* d = nullptr;
  void* s = nullptr;
  if (cudaGetSymbolAddress(&d, g_delta_scratch) != cudaSuccess) return false;
  if (cudaGetSymbolAddress(&s, g_status_scratch) != cudaSuccess) return false;
  g_delta_ptr[device] = static_cast<float*>(d);
  g_status_ptr[device] = static_cast<bux::Status*>(s);
  return true;
}

int fail(int code, const char* text, const char** message) {
  if (message) *message = text;
  return code;
}

}  // namespace

extern "C" int bux_attn_bwd_static(const void* q, const void* k, const void* v, const void* o,
                                   const void* d_o, const float* lse, float* dq, void* dk, void* dv,
                                   const float* sinks, float* dsinks, int B, int T, int S, int H,
                                   int G, int D, float scale, int causal, int window,
                                   void* cuda_stream, const char** message) {
  if (message) *message = "ok";
  if (B <= 0 || T <= 0 || S <= 0 || H <= 0 || G <= 0 || H % G != 0 || (D != 64 && D != 128))
    return fail(2, "unsupported shape: head_dim is 64 or 128 and query heads a multiple of kv heads", message);
  const long rows = (long)B * H * T;
  if (rows > BUX_ATTN_BWD_STATIC_MAX_ROWS)
    return fail(1, "batch * heads * length exceeds the built-in scratch (BUX_ATTN_BWD_STATIC_MAX_ROWS)", message);
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return fail(3, "no usable current device", message);
  if (!resolve(device)) return fail(3, "the scratch array's device address could not be resolved", message);
  cudaStream_t stream = static_cast<cudaStream_t>(cuda_stream);
  // dq is accumulated with atomics and dsinks likewise: both start from zero.
  if (cudaMemsetAsync(dq, 0, sizeof(float) * (size_t)B * T * H * D, stream) != cudaSuccess)
    return fail(4, "clearing dq failed", message);
  if (dsinks != nullptr && cudaMemsetAsync(dsinks, 0, sizeof(float) * H, stream) != cudaSuccess)
    return fail(4, "clearing dsinks failed", message);
  bux::AttnArgs a;
  a.q = q; a.k = k; a.v = v; a.o = const_cast<void*>(o); a.lse = const_cast<float*>(lse);
  a.d_o = d_o; a.dq = dq; a.dk = dk; a.dv = dv;
  a.delta = g_delta_ptr[device];
  a.sinks = sinks; a.dsinks = dsinks;
  a.B = B; a.T = T; a.S = S; a.H = H; a.G = G; a.D = D;
  a.scale = scale; a.causal = causal != 0; a.window = window;
  a.status = g_status_ptr[device];
  const char* err = bux::attn_bwd_launch(a, stream);
  if (err != nullptr) return fail(4, err, message);
  return 0;
}

extern "C" int bux_attn_bwd_static_status(unsigned int* code, unsigned int* count, int clear) {
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return 3;
  if (!resolve(device)) return 3;
  bux::Status host{0u, 0u};
  // a blocking copy on the legacy default stream: it returns after the work queued before it
  if (cudaMemcpy(&host, g_status_ptr[device], sizeof(host), cudaMemcpyDeviceToHost) != cudaSuccess) return 4;
  if (code) *code = host.code;
  if (count) *count = host.count;
  if (clear && (host.code != 0u || host.count != 0u) &&
      cudaMemset(g_status_ptr[device], 0, sizeof(host)) != cudaSuccess)
    return 4;
  return 0;
}
