// Host-visible types of the chunkwise-recurrence kernel (scan_sm100.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace bux {

struct Status;

// The serial part of a chunked linear recurrence for `bh` independent (row, head) pairs of
// `n_chunks` chunks of 64 positions, head dims padded to 128. All matrix operands are bf16,
// row-major, one block of rows per (pair, chunk):
//   a1   [bh*n*128, 128]  rows 0-63 multiply the state into X, rows 64-127 into the output
//   aux1 [bh*n*128, 64]   the same two blocks' factors of V
//   aux3 [bh*n*64, 64]    the output's factor of X (null: no output chain)
//   a4   [bh*n*128, 128]  rows 0-63 pair with V, rows 64-127 with X in the state's update
//   v    [bh*n*64, 128]
//   lam  [bh*n, 128] fp32 decay of the state over the chunk;  s0 [bh, 128, 128] fp32 or null
// Outputs: out / x_out [bh*n*64, 128] bf16 (either may be null), states [bh*n, 128, 128] bf16 (the
// state each chunk starts from; may be null), s_last [bh, 128, 128] fp32. `reverse` walks the
// chunks from the last to the first.
struct ScanArgs {
  const void* a1 = nullptr; const void* aux1 = nullptr; const void* aux3 = nullptr;
  const void* a4 = nullptr; const void* v = nullptr;
  const float* lam = nullptr; const float* s0 = nullptr;
  void* out = nullptr; void* x_out = nullptr; void* states = nullptr; float* s_last = nullptr;
  int bh = 0, n_chunks = 0, dk = 128, dv = 128;
  bool reverse = false;
  Status* status = nullptr;
};

const char* chunk_scan_launch(const ScanArgs& a, cudaStream_t stream);

}  // namespace bux
