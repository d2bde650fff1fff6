// torch.ops.bux_b200.* : thin tensor-checking wrappers around the CUDA launchers.
// Registered with TORCH_LIBRARY so the shared object is loaded with
// torch.ops.load_library and needs no Python headers.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "attention_sm100.h"
#include "comm_sm100.h"
#include "elementwise.h"
#include "gemm_sm100.h"
#include "scan_sm100.h"

namespace {

using at::Tensor;

cudaStream_t stream_of(const Tensor& t) {
  return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}
void check_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor");
  TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}
bux::Status* status_ptr(const c10::optional<Tensor>& st) {
  if (!st.has_value()) return nullptr;
  TORCH_CHECK(st->is_cuda() && st->scalar_type() == at::kInt && st->numel() >= 2, "status: int32[2] on the device");
  return reinterpret_cast<bux::Status*>(st->data_ptr());
}
const float* opt_f32(const c10::optional<Tensor>& t) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous(), "expected a contiguous fp32 CUDA tensor");
  return t->data_ptr<float>();
}
const int* opt_i32(const c10::optional<Tensor>& t) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous(), "expected a contiguous int32 CUDA tensor");
  return t->data_ptr<int>();
}

// ------------------------------------------------------------------ GEMM
// c (+)= a · b^T.  kind 0 = bf16, 1 = mxfp8 (a/b uint8 e4m3 bytes, sfa/sfb tiled scales).
// a_mn / b_mn: operand stored transposed ([K, M] / [K, N]).  mode: 0 dense, 1 grouped rows
// (b is [groups*N, K] or, MN-major, [groups*K, N]), 2 grouped contraction.
void gemm(const Tensor& a, const Tensor& b, Tensor& c, const c10::optional<Tensor>& sfa,
          const c10::optional<Tensor>& sfb, const c10::optional<Tensor>& group_offsets,
          const c10::optional<Tensor>& status, int64_t kind, int64_t mode, int64_t M, int64_t N,
          int64_t K, int64_t k_total, int64_t groups, bool a_mn, bool b_mn, int64_t out_kind,
          int64_t bn, int64_t sms, const c10::optional<Tensor>& wait_flags, int64_t wait_epoch,
          int64_t wait_rows, int64_t m_rotate, bool wait_on_k, bool wait_on_n) {
  check_cuda(a, "a"); check_cuda(b, "b"); check_cuda(c, "c");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2, "a and b are 2-D views");
  c10::cuda::CUDAGuard guard(a.device());
  bux::GemmArgs g;
  g.kind = (int)kind; g.mode = (int)mode; g.bn = (int)bn; g.out_kind = (int)out_kind;
  g.a_mn = a_mn; g.b_mn = b_mn;
  const int elem = kind == bux::KIND_BF16 ? 2 : 1;
  TORCH_CHECK((int)a.element_size() == elem && (int)b.element_size() == elem, "operand dtype does not match kind");
  g.a = a.data_ptr(); g.a_outer = a.size(0); g.a_inner = a.size(1); g.lda_bytes = a.stride(0) * elem;
  g.b = b.data_ptr(); g.b_outer = b.size(0); g.b_inner = b.size(1); g.ldb_bytes = b.stride(0) * elem;
  if (kind == bux::KIND_MXFP8) {
    TORCH_CHECK(sfa.has_value() && sfb.has_value(), "mxfp8 needs scale tensors");
    g.sfa = reinterpret_cast<const uint8_t*>(sfa->data_ptr());
    g.sfb = reinterpret_cast<const uint8_t*>(sfb->data_ptr());
  }
  g.c = c.data_ptr(); g.ldc = (int)c.stride(c.dim() - 2);
  TORCH_CHECK((out_kind == bux::OUT_BF16 || out_kind == bux::OUT_BF16_ACC) ? c.scalar_type() == at::kBFloat16
                                                                            : c.scalar_type() == at::kFloat,
              "c dtype does not match out_kind");
  g.M = (int)M; g.N = (int)N; g.K = (int)K; g.k_total = (int)k_total; g.groups = (int)groups;
  g.group_offsets = opt_i32(group_offsets);
  TORCH_CHECK(mode == bux::MODE_DENSE || g.group_offsets != nullptr, "grouped modes need group_offsets");
  g.status = status_ptr(status);
  g.sms = (int)sms;
  if (wait_flags.has_value()) {
    g.wait_flags = opt_i32(wait_flags); g.wait_world = (int)wait_flags->numel(); g.wait_epoch = (int)wait_epoch;
    g.wait_rows = (int)wait_rows; g.wait_on_k = wait_on_k; g.wait_on_n = wait_on_n;
  }
  g.m_rotate = (int)m_rotate;
  const char* err = bux::gemm_launch(g, stream_of(a));
  TORCH_CHECK(err == nullptr, "bux gemm: ", err);
}

// ------------------------------------------------------------------ norms
void rmsnorm_fwd(const Tensor& x, const c10::optional<Tensor>& w, Tensor& y, Tensor& rstd, double eps) {
  check_cuda(x, "x"); check_cuda(y, "y");
  const int d = (int)x.size(-1);
  TORCH_CHECK(d % 8 == 0 && x.scalar_type() == at::kBFloat16, "rmsnorm: bf16, width % 8 == 0");
  c10::cuda::CUDAGuard guard(x.device());
  bux::rmsnorm_fwd(x.data_ptr(), opt_f32(w), y.data_ptr(), rstd.data_ptr<float>(), x.numel() / d, d, (float)eps, stream_of(x));
}
void rmsnorm_bwd(const Tensor& x, const c10::optional<Tensor>& w, const Tensor& dy, const Tensor& rstd,
                 Tensor& dx, const c10::optional<Tensor>& dw) {
  check_cuda(x, "x"); check_cuda(dy, "dy"); check_cuda(dx, "dx");
  const int d = (int)x.size(-1);
  c10::cuda::CUDAGuard guard(x.device());
  float* dwp = dw.has_value() ? dw->data_ptr<float>() : nullptr;
  bux::rmsnorm_bwd(x.data_ptr(), opt_f32(w), dy.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), dwp, x.numel() / d, d, stream_of(x));
}
// x viewed as [tokens, heads, D] with token stride stride_x (elements); y likewise.
void norm_rope(bool bwd, const Tensor& x, const c10::optional<Tensor>& w, const Tensor& cos, const Tensor& sin,
               Tensor& y, const c10::optional<Tensor>& rstd, const c10::optional<Tensor>& dy,
               const c10::optional<Tensor>& dw, int64_t tokens, int64_t heads, int64_t D,
               int64_t stride_x, int64_t stride_y, double eps) {
  TORCH_CHECK(x.is_cuda() && y.is_cuda() && x.scalar_type() == at::kBFloat16, "norm_rope: bf16 CUDA tensors");
  c10::cuda::CUDAGuard guard(x.device());
  float* rs = rstd.has_value() ? rstd->data_ptr<float>() : nullptr;
  float* dwp = dw.has_value() ? dw->data_ptr<float>() : nullptr;
  const void* dyp = dy.has_value() ? dy->data_ptr() : nullptr;
  const char* err = bux::norm_rope(bwd, x.data_ptr(), opt_f32(w), cos.data_ptr<float>(), sin.data_ptr<float>(), y.data_ptr(), rs, dyp, dwp,
                                   tokens, (int)heads, (int)D, stride_x, stride_y, (float)eps, stream_of(x));
  TORCH_CHECK(err == nullptr, err);
}

// ------------------------------------------------------------------ GLU
void glu_fwd(const Tensor& h, Tensor& out, const c10::optional<Tensor>& row_scale, int64_t kind, double limit, double up_offset) {
  check_cuda(h, "h"); check_cuda(out, "out");
  const int f = (int)out.size(-1);
  TORCH_CHECK(h.size(-1) == 2 * f && f % 8 == 0, "glu: h is [rows, 2f], f % 8 == 0");
  c10::cuda::CUDAGuard guard(h.device());
  bux::glu_fwd(h.data_ptr(), out.data_ptr(), opt_f32(row_scale), out.numel() / f, f, (int)kind, (float)limit, (float)up_offset, stream_of(h));
}
void glu_bwd(const Tensor& h, const Tensor& dout, Tensor& dh, const c10::optional<Tensor>& row_scale,
             const c10::optional<Tensor>& d_row_scale, int64_t kind, double limit, double up_offset) {
  check_cuda(h, "h"); check_cuda(dout, "dout"); check_cuda(dh, "dh");
  const int f = (int)dout.size(-1);
  c10::cuda::CUDAGuard guard(h.device());
  float* drs = d_row_scale.has_value() ? d_row_scale->data_ptr<float>() : nullptr;
  bux::glu_bwd(h.data_ptr(), dout.data_ptr(), dh.data_ptr(), opt_f32(row_scale), drs, dout.numel() / f, f, (int)kind, (float)limit, (float)up_offset, stream_of(h));
}

// ------------------------------------------------------------------ MXFP8 quantiser
void quant_mxfp8(const Tensor& x, const c10::optional<Tensor>& row_index, const c10::optional<Tensor>& row_scale,
                 const c10::optional<Tensor>& q_row,
                 const c10::optional<Tensor>& sf_row, const c10::optional<Tensor>& q_col,
                 const c10::optional<Tensor>& sf_col, int64_t rows, int64_t cols, int64_t ld_col,
                 int64_t batch, int64_t x_batch_stride) {
  TORCH_CHECK(x.is_cuda() && x.scalar_type() == at::kBFloat16 && x.stride(-1) == 1, "quant: bf16 rows");
  TORCH_CHECK(cols % 32 == 0, "quant: columns % 32 == 0");
  c10::cuda::CUDAGuard guard(x.device());
  uint8_t* qr = q_row.has_value() ? reinterpret_cast<uint8_t*>(q_row->data_ptr()) : nullptr;
  uint8_t* sr = sf_row.has_value() ? reinterpret_cast<uint8_t*>(sf_row->data_ptr()) : nullptr;
  uint8_t* qc = q_col.has_value() ? reinterpret_cast<uint8_t*>(q_col->data_ptr()) : nullptr;
  uint8_t* sc = sf_col.has_value() ? reinterpret_cast<uint8_t*>(sf_col->data_ptr()) : nullptr;
  TORCH_CHECK(qc == nullptr || ld_col % 32 == 0, "quant: transposed copy needs a row count padded to 32");
  bux::quant_mxfp8(x.data_ptr(), x.stride(-2), opt_i32(row_index), opt_f32(row_scale), qr, sr, qc, sc, rows, (int)cols, ld_col, (int)batch, x_batch_stride, stream_of(x));
}

void quant_mxfp8_glu(const Tensor& h, const c10::optional<Tensor>& dout, const c10::optional<Tensor>& row_scale,
                     const c10::optional<Tensor>& q_row,
                     const c10::optional<Tensor>& sf_row, const c10::optional<Tensor>& q_col,
                     const c10::optional<Tensor>& sf_col, int64_t ld_col, int64_t kind, double limit, double up_offset) {
  TORCH_CHECK(h.is_cuda() && h.scalar_type() == at::kBFloat16 && h.dim() == 2 && h.is_contiguous(), "quant_glu: contiguous bf16 h [rows, 2f]");
  const int64_t rows = h.size(0), f = h.size(1) / 2;
  TORCH_CHECK(f % 32 == 0, "quant_glu: f % 32 == 0");
  const void* dp = nullptr;
  if (dout.has_value()) {
    TORCH_CHECK(dout->is_cuda() && dout->scalar_type() == at::kBFloat16 && dout->is_contiguous() &&
                dout->size(0) == rows && dout->size(1) == f, "quant_glu: contiguous bf16 dout [rows, f]");
    TORCH_CHECK(f % 128 == 0, "quant_glu: the gradient wants f % 128 == 0");
    dp = dout->data_ptr();
  }
  c10::cuda::CUDAGuard guard(h.device());
  uint8_t* qr = q_row.has_value() ? reinterpret_cast<uint8_t*>(q_row->data_ptr()) : nullptr;
  uint8_t* sr = sf_row.has_value() ? reinterpret_cast<uint8_t*>(sf_row->data_ptr()) : nullptr;
  uint8_t* qc = q_col.has_value() ? reinterpret_cast<uint8_t*>(q_col->data_ptr()) : nullptr;
  uint8_t* sc = sf_col.has_value() ? reinterpret_cast<uint8_t*>(sf_col->data_ptr()) : nullptr;
  TORCH_CHECK(qc == nullptr || ld_col % 32 == 0, "quant_glu: transposed copy needs a row count padded to 32");
  if (row_scale.has_value())
    TORCH_CHECK(row_scale->is_cuda() && row_scale->scalar_type() == at::kFloat && row_scale->is_contiguous() &&
                row_scale->numel() >= rows && !dout.has_value(), "quant_glu: row_scale is fp32 [rows], activation only");
  bux::quant_mxfp8_glu(h.data_ptr(), dp, opt_f32(row_scale), qr, sr, qc, sc, rows, (int)f, ld_col, (int)kind,
                       (float)limit, (float)up_offset, stream_of(h));
}

void quant_nvfp4(const Tensor& x, const Tensor& tensor_scale, Tensor& packed, Tensor& scales) {
  check_cuda(x, "x");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2 && x.size(1) % 16 == 0,
              "quant_nvfp4: contiguous bf16 [rows, cols], cols % 16 == 0");
  TORCH_CHECK(tensor_scale.is_cuda() && tensor_scale.scalar_type() == at::kFloat && tensor_scale.numel() == 1,
              "quant_nvfp4: the tensor scale is one fp32 value on the device");
  TORCH_CHECK(packed.numel() == x.numel() / 2 && scales.numel() == x.numel() / 16 && packed.element_size() == 1 &&
              scales.element_size() == 1, "quant_nvfp4: packed [rows, cols/2] and scales [rows, cols/16] bytes");
  c10::cuda::CUDAGuard guard(x.device());
  bux::quant_nvfp4(x.data_ptr(), tensor_scale.data_ptr<float>(), reinterpret_cast<uint8_t*>(packed.data_ptr()),
                   reinterpret_cast<uint8_t*>(scales.data_ptr()), x.size(0), (int)x.size(1), stream_of(x));
}

// ------------------------------------------------------------------ loss / optimiser / MoE rows
void ce_fwd_bwd(Tensor& logits, const Tensor& targets, const c10::optional<Tensor>& mask, Tensor& loss,
                const c10::optional<Tensor>& logz, double grad_scale, double z_weight, double softcap) {
  check_cuda(logits, "logits");
  TORCH_CHECK(logits.scalar_type() == at::kBFloat16 && logits.size(-1) % 8 == 0, "ce: bf16 logits, vocab % 8 == 0");
  c10::cuda::CUDAGuard guard(logits.device());
  float* lz = logz.has_value() ? logz->data_ptr<float>() : nullptr;
  bux::ce_fwd_bwd(logits.data_ptr(), targets.data_ptr<int>(), opt_f32(mask), loss.data_ptr<float>(), lz,
                  logits.size(0), (int)logits.size(1), logits.stride(0), (float)grad_scale, (float)z_weight, (float)softcap, stream_of(logits));
}
void adamw(Tensor& p, const Tensor& g, Tensor& m, Tensor& v, const c10::optional<Tensor>& m_sf,
           const c10::optional<Tensor>& v_sf, const c10::optional<Tensor>& shadow,
           const c10::optional<Tensor>& grad_scale, double lr, double b1, double b2, double eps,
           double wd, double bc1, double bc2, double grad_scale_const) {
  check_cuda(p, "p"); check_cuda(g, "g"); check_cuda(m, "m"); check_cuda(v, "v");
  c10::cuda::CUDAGuard guard(p.device());
  int mom = m.scalar_type() == at::kFloat ? bux::MOM_F32 : m.scalar_type() == at::kBFloat16 ? bux::MOM_BF16 : bux::MOM_FP8;
  uint8_t* msf = m_sf.has_value() ? reinterpret_cast<uint8_t*>(m_sf->data_ptr()) : nullptr;
  uint8_t* vsf = v_sf.has_value() ? reinterpret_cast<uint8_t*>(v_sf->data_ptr()) : nullptr;
  TORCH_CHECK(mom != bux::MOM_FP8 || (msf && vsf), "8-bit moments need scale tensors");
  void* sh = shadow.has_value() ? shadow->data_ptr() : nullptr;
  const char* err = bux::adamw(p.data_ptr(), p.scalar_type() == at::kBFloat16, g.data_ptr(), g.scalar_type() == at::kBFloat16,
                               m.data_ptr(), v.data_ptr(), msf, vsf, mom, sh, p.numel(), (float)lr, (float)b1, (float)b2,
                               (float)eps, (float)wd, (float)bc1, (float)bc2, opt_f32(grad_scale), (float)grad_scale_const, stream_of(p));
  TORCH_CHECK(err == nullptr, err);
}
void sumsq(const Tensor& g, Tensor& out) {
  check_cuda(g, "g");
  c10::cuda::CUDAGuard guard(g.device());
  bux::sumsq(g.data_ptr(), g.scalar_type() == at::kBFloat16, g.numel(), out.data_ptr<float>(), stream_of(g));
}
void topk_rows(const Tensor& scores, Tensor& idx) {
  check_cuda(scores, "scores"); check_cuda(idx, "idx");
  TORCH_CHECK(scores.scalar_type() == at::kFloat && scores.dim() == 2 && scores.is_contiguous(), "topk_rows: contiguous fp32 [rows, n]");
  TORCH_CHECK(idx.scalar_type() == at::kLong && idx.is_contiguous() && idx.size(0) == scores.size(0), "topk_rows: int64 [rows, k]");
  TORCH_CHECK(idx.size(1) <= scores.size(1), "topk_rows: k <= n");
  c10::cuda::CUDAGuard guard(scores.device());
  const char* err = bux::topk_rows(scores.data_ptr<float>(), reinterpret_cast<long*>(idx.data_ptr<int64_t>()), scores.size(0),
                                   (int)scores.size(1), (int)idx.size(1), stream_of(scores));
  TORCH_CHECK(err == nullptr, err);
}
void gather_rows(const Tensor& x, const Tensor& index, Tensor& out) {
  check_cuda(x, "x"); check_cuda(out, "out");
  c10::cuda::CUDAGuard guard(x.device());
  bux::gather_rows(x.data_ptr(), index.data_ptr<int>(), out.data_ptr(), out.size(0), (int)out.size(1), stream_of(x));
}
void combine_bwd(const c10::optional<Tensor>& y, const Tensor& dout, const Tensor& pos, const c10::optional<Tensor>& w,
                 const c10::optional<Tensor>& dy, const c10::optional<Tensor>& dw) {
  check_cuda(dout, "dout");
  c10::cuda::CUDAGuard guard(dout.device());
  const void* yp = y.has_value() ? y->data_ptr() : nullptr;
  float* dwp = (dw.has_value() && yp) ? dw->data_ptr<float>() : nullptr;
  bux::combine_bwd(yp, dout.data_ptr(), pos.data_ptr<int>(), opt_f32(w), dy.has_value() ? dy->data_ptr() : nullptr, dwp, pos.numel(), (int)pos.size(1), (int)dout.size(1), stream_of(dout));
}
void combine_rows(const Tensor& y, const Tensor& pos, const c10::optional<Tensor>& w, Tensor& out) {
  check_cuda(y, "y"); check_cuda(out, "out");
  c10::cuda::CUDAGuard guard(y.device());
  bux::combine_rows(y.data_ptr(), pos.data_ptr<int>(), opt_f32(w), out.data_ptr(), out.size(0), (int)pos.size(1), (int)out.size(1), stream_of(y));
}

// ------------------------------------------------------------------ attention
const int* doc_bounds(const c10::optional<Tensor>& t, int64_t numel, const char* name) {
  if (!t.has_value()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kInt && t->is_contiguous() && t->numel() == numel,
              "bux attention: ", name, " is a contiguous int32 tensor with one entry per position");
  return t->data_ptr<int>();
}

void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& o, Tensor& lse,
              const c10::optional<Tensor>& sinks, const c10::optional<Tensor>& status,
              double scale, bool causal, int64_t window, const c10::optional<Tensor>& row_lo) {
  check_cuda(q, "q"); check_cuda(k, "k"); check_cuda(v, "v"); check_cuda(o, "o");
  c10::cuda::CUDAGuard guard(q.device());
  bux::AttnArgs a;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr(); a.lse = lse.data_ptr<float>();
  a.sinks = opt_f32(sinks);
  a.B = (int)q.size(0); a.T = (int)q.size(1); a.H = (int)q.size(2); a.D = (int)q.size(3);
  a.S = (int)k.size(1); a.G = (int)k.size(2);
  a.scale = (float)scale; a.causal = causal; a.window = (int)window;
  a.status = status_ptr(status);
  a.row_lo = doc_bounds(row_lo, q.size(0) * q.size(1), "row_lo");
  TORCH_CHECK(a.row_lo == nullptr || (causal && a.T == a.S), "bux attention: documents need causal self-attention");
  const char* err = bux::attn_fwd_launch(a, stream_of(q));
  TORCH_CHECK(err == nullptr, "bux attention: ", err);
}
void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& d_o,
              const Tensor& lse, Tensor& dq, Tensor& dk, Tensor& dv, Tensor& delta,
              const c10::optional<Tensor>& sinks, const c10::optional<Tensor>& dsinks,
              const c10::optional<Tensor>& status, double scale, bool causal, int64_t window,
              const c10::optional<Tensor>& row_lo, const c10::optional<Tensor>& key_hi,
              const c10::optional<Tensor>& phase_cycles) {
  check_cuda(q, "q"); check_cuda(d_o, "do");
  c10::cuda::CUDAGuard guard(q.device());
  bux::AttnArgs a;
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr(); a.o = o.data_ptr(); a.lse = lse.data_ptr<float>();
  a.d_o = d_o.data_ptr(); a.dq = dq.data_ptr(); a.dk = dk.data_ptr(); a.dv = dv.data_ptr(); a.delta = delta.data_ptr<float>();
  a.sinks = opt_f32(sinks);
  a.dsinks = dsinks.has_value() ? dsinks->data_ptr<float>() : nullptr;
  a.B = (int)q.size(0); a.T = (int)q.size(1); a.H = (int)q.size(2); a.D = (int)q.size(3);
  a.S = (int)k.size(1); a.G = (int)k.size(2);
  a.scale = (float)scale; a.causal = causal; a.window = (int)window;
  a.status = status_ptr(status);
  a.row_lo = doc_bounds(row_lo, q.size(0) * q.size(1), "row_lo");
  a.key_hi = doc_bounds(key_hi, k.size(0) * k.size(1), "key_hi");
  TORCH_CHECK((a.row_lo == nullptr) == (a.key_hi == nullptr), "bux attention backward: row_lo and key_hi go together");
  TORCH_CHECK(a.row_lo == nullptr || (causal && a.T == a.S), "bux attention: documents need causal self-attention");
  if (phase_cycles.has_value()) {
    TORCH_CHECK(phase_cycles->is_cuda() && phase_cycles->scalar_type() == at::kInt && phase_cycles->numel() >= 32 &&
                    phase_cycles->is_contiguous(), "bux attention backward: phase_cycles is int32[32] on the device");
    a.phase_cycles = reinterpret_cast<unsigned int*>(phase_cycles->data_ptr<int>());
  }
  const char* err = bux::attn_bwd_launch(a, stream_of(q));
  TORCH_CHECK(err == nullptr, "bux attention backward: ", err);
}

// ------------------------------------------------------------------ causal depthwise convolution
void causal_conv(bool bwd, const Tensor& in, const Tensor& w, const c10::optional<Tensor>& bias,
                 const c10::optional<Tensor>& position, Tensor& out) {
  check_cuda(in, "in"); check_cuda(out, "out");
  TORCH_CHECK(in.dim() == 3 && in.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 &&
                  out.sizes() == in.sizes(), "causal_conv: [B, T, C] bf16 in and out");
  TORCH_CHECK(w.is_cuda() && w.scalar_type() == at::kFloat && w.is_contiguous() && w.dim() == 2 && w.size(0) == in.size(2),
              "causal_conv: w is fp32 [C, taps]");
  TORCH_CHECK(!position.has_value() || position->numel() == in.size(0) * in.size(1), "causal_conv: position is int32 [B, T]");
  c10::cuda::CUDAGuard guard(in.device());
  const char* err = bux::causal_conv(bwd, in.data_ptr(), w.data_ptr<float>(), opt_f32(bias), opt_i32(position), out.data_ptr(),
                                     (int)in.size(0), (int)in.size(1), (int)in.size(2), (int)w.size(1), stream_of(in));
  TORCH_CHECK(err == nullptr, "bux ", err);
}
void causal_conv_wgrad(const Tensor& x, const Tensor& dy, const c10::optional<Tensor>& position, Tensor& dw,
                       const c10::optional<Tensor>& db) {
  check_cuda(x, "x"); check_cuda(dy, "dy"); check_cuda(dw, "dw");
  TORCH_CHECK(x.dim() == 3 && x.scalar_type() == at::kBFloat16 && dy.scalar_type() == at::kBFloat16 && dy.sizes() == x.sizes(),
              "causal_conv_wgrad: [B, T, C] bf16 x and dy");
  TORCH_CHECK(dw.scalar_type() == at::kFloat && dw.dim() == 2 && dw.size(0) == x.size(2), "causal_conv_wgrad: dw is fp32 [C, taps]");
  c10::cuda::CUDAGuard guard(x.device());
  float* dbp = nullptr;
  if (db.has_value()) {
    TORCH_CHECK(db->is_cuda() && db->scalar_type() == at::kFloat && db->numel() == x.size(2), "causal_conv_wgrad: db is fp32 [C]");
    dbp = db->data_ptr<float>();
  }
  const char* err = bux::causal_conv_wgrad(x.data_ptr(), dy.data_ptr(), opt_i32(position), dw.data_ptr<float>(), dbp,
                                           (int)x.size(0), (int)x.size(1), (int)x.size(2), (int)dw.size(1), stream_of(x));
  TORCH_CHECK(err == nullptr, "bux ", err);
}

// ------------------------------------------------------------------ chunkwise recurrence
void chunk_scan(const Tensor& a1, const Tensor& aux1, const c10::optional<Tensor>& aux3, const Tensor& a4, const Tensor& v,
                const Tensor& lam, const c10::optional<Tensor>& s0, const c10::optional<Tensor>& out,
                const c10::optional<Tensor>& x_out, const c10::optional<Tensor>& states, Tensor& s_last,
                const c10::optional<Tensor>& status, int64_t bh, int64_t n_chunks, bool reverse) {
  check_cuda(a1, "a1"); check_cuda(aux1, "aux1"); check_cuda(a4, "a4"); check_cuda(v, "v"); check_cuda(lam, "lam");
  check_cuda(s_last, "s_last");
  auto bf16 = [](const Tensor& t, int64_t numel, const char* name) {
    TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.is_contiguous() && t.numel() == numel,
                "chunk_scan: ", name, " must be contiguous bf16 of ", numel, " elements");
  };
  const int64_t chunks = bh * n_chunks;
  TORCH_CHECK(chunks * 128 < (int64_t(1) << 31), "chunk_scan: too many rows for one launch");
  bf16(a1, chunks * 128 * 128, "a1"); bf16(aux1, chunks * 128 * 64, "aux1"); bf16(a4, chunks * 128 * 128, "a4");
  bf16(v, chunks * 64 * 128, "v");
  if (aux3.has_value()) bf16(*aux3, chunks * 64 * 64, "aux3");
  if (out.has_value()) bf16(*out, chunks * 64 * 128, "out");
  if (x_out.has_value()) bf16(*x_out, chunks * 64 * 128, "x_out");
  if (states.has_value()) bf16(*states, chunks * 128 * 128, "states");
  TORCH_CHECK(lam.scalar_type() == at::kFloat && lam.numel() == chunks * 128, "chunk_scan: lam is fp32 [bh*n, 128]");
  TORCH_CHECK(s_last.scalar_type() == at::kFloat && s_last.numel() == bh * 128 * 128, "chunk_scan: s_last is fp32 [bh, 128, 128]");
  TORCH_CHECK(!s0.has_value() || s0->numel() == bh * 128 * 128, "chunk_scan: s0 is fp32 [bh, 128, 128]");
  c10::cuda::CUDAGuard guard(a1.device());
  bux::ScanArgs a;
  a.a1 = a1.data_ptr(); a.aux1 = aux1.data_ptr(); a.aux3 = aux3.has_value() ? aux3->data_ptr() : nullptr;
  a.a4 = a4.data_ptr(); a.v = v.data_ptr(); a.lam = lam.data_ptr<float>(); a.s0 = opt_f32(s0);
  a.out = out.has_value() ? out->data_ptr() : nullptr;
  a.x_out = x_out.has_value() ? x_out->data_ptr() : nullptr;
  a.states = states.has_value() ? states->data_ptr() : nullptr;
  a.s_last = s_last.data_ptr<float>();
  a.bh = (int)bh; a.n_chunks = (int)n_chunks; a.reverse = reverse; a.status = status_ptr(status);
  const char* err = bux::chunk_scan_launch(a, stream_of(a1));
  TORCH_CHECK(err == nullptr, "bux chunk_scan: ", err);
}

// ------------------------------------------------------------------ expert-parallel exchange
const uint64_t* u64_ptr(const Tensor& t) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kLong && t.is_contiguous(), "expected an int64 CUDA table of addresses");
  return reinterpret_cast<const uint64_t*>(t.data_ptr());
}
void ep_push_rows(const Tensor& x, const Tensor& src_token, const Tensor& dst_rank, const Tensor& dst_row,
                  const c10::optional<Tensor>& row_scale, const Tensor& peer_base, int64_t sms,
                  const c10::optional<Tensor>& peer_scale) {
  check_cuda(x, "x");
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(!peer_scale.has_value() || row_scale.has_value(), "ep_push_rows: peer_scale needs row_scale");
  bux::ep_push_rows(x.data_ptr(), src_token.data_ptr<int>(), dst_rank.data_ptr<int>(), dst_row.data_ptr<int>(),
                    opt_f32(row_scale), u64_ptr(peer_base), peer_scale.has_value() ? u64_ptr(*peer_scale) : nullptr,
                    dst_row.numel(), (int)x.size(-1), (int)sms, stream_of(x));
}
void ep_push_rows_mx(const Tensor& x, const Tensor& rank_of, const Tensor& row_of, const c10::optional<Tensor>& w,
                     const Tensor& peer_q, const Tensor& peer_sf, const c10::optional<Tensor>& peer_scale, int64_t sms) {
  check_cuda(x, "x");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.is_contiguous() && x.dim() == 2 && x.size(1) % 128 == 0,
              "ep_push_rows_mx: contiguous bf16 rows of a multiple of 128 columns");
  TORCH_CHECK(row_of.dim() == 2 && row_of.size(0) == x.size(0) && row_of.size(1) <= 32 && row_of.is_contiguous() &&
                  rank_of.is_contiguous() && rank_of.sizes() == row_of.sizes(),
              "ep_push_rows_mx: rank_of / row_of are [tokens, k <= 32] int32");
  TORCH_CHECK(!w.has_value() || (w->is_contiguous() && w->numel() == row_of.numel()), "ep_push_rows_mx: w is [tokens, k] fp32");
  c10::cuda::CUDAGuard guard(x.device());
  bux::ep_push_rows_mx(x.data_ptr(), rank_of.data_ptr<int>(), row_of.data_ptr<int>(), opt_f32(w), u64_ptr(peer_q),
                       u64_ptr(peer_sf), peer_scale.has_value() ? u64_ptr(*peer_scale) : nullptr, x.size(0),
                       (int)row_of.size(1), (int)x.size(1), (int)sms, stream_of(x));
}
void requant_mxfp8_cols(const Tensor& q, const Tensor& sf, Tensor& q_col, Tensor& sf_col, int64_t rows, int64_t cols,
                        int64_t ld_col) {
  check_cuda(q, "q"); check_cuda(sf, "sf");
  TORCH_CHECK(q.is_contiguous() && q.element_size() == 1 && q.numel() >= rows * cols && cols % 32 == 0 && ld_col % 32 == 0,
              "requant_mxfp8_cols: contiguous e4m3 bytes [rows, cols], cols and the padded row count multiples of 32");
  c10::cuda::CUDAGuard guard(q.device());
  bux::requant_mxfp8_cols(reinterpret_cast<const uint8_t*>(q.data_ptr()), reinterpret_cast<const uint8_t*>(sf.data_ptr()),
                          reinterpret_cast<uint8_t*>(q_col.data_ptr()), reinterpret_cast<uint8_t*>(sf_col.data_ptr()),
                          rows, (int)cols, ld_col, stream_of(q));
}
void row_dots(const Tensor& a, const Tensor& b, Tensor& out) {
  check_cuda(a, "a"); check_cuda(b, "b");
  TORCH_CHECK(a.scalar_type() == at::kBFloat16 && b.scalar_type() == at::kBFloat16 && a.is_contiguous() && b.is_contiguous() &&
              a.dim() == 2 && a.sizes() == b.sizes() && a.size(1) % 8 == 0, "row_dots: two contiguous bf16 [rows, d], d % 8 == 0");
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.numel() >= a.size(0), "row_dots: fp32 out of at least `rows`");
  c10::cuda::CUDAGuard guard(a.device());
  bux::row_dots(a.data_ptr(), b.data_ptr(), out.data_ptr<float>(), a.size(0), (int)a.size(1), stream_of(a));
}
void ep_pull_scalar(const Tensor& peer_base, const Tensor& rank_of, const Tensor& row_of, Tensor& out,
                    const c10::optional<Tensor>& flags, int64_t epoch, const c10::optional<Tensor>& status, double limit_s) {
  check_cuda(out, "out");
  TORCH_CHECK(out.scalar_type() == at::kFloat && out.numel() == row_of.numel(), "ep_pull_scalar: fp32 out, one per pick");
  c10::cuda::CUDAGuard guard(out.device());
  const int* fl = opt_i32(flags);
  bux::ep_pull_scalar(u64_ptr(peer_base), rank_of.data_ptr<int>(), row_of.data_ptr<int>(), out.data_ptr<float>(), row_of.numel(),
                      fl, fl ? (int)flags->numel() : 0, (int)epoch, (uint64_t)(limit_s * 1e9), status_ptr(status), stream_of(out));
}
void ep_signal(const Tensor& peer_flags, int64_t channel, int64_t world, int64_t my_rank, int64_t epoch) {
  c10::cuda::CUDAGuard guard(peer_flags.device());
  bux::ep_signal(u64_ptr(peer_flags), (int)channel, (int)world, (int)my_rank, (int)epoch, stream_of(peer_flags));
}
void ep_pull_combine(const Tensor& peer_base, const Tensor& rank_of, const Tensor& row_of, const c10::optional<Tensor>& w,
                     Tensor& out, const c10::optional<Tensor>& flags, int64_t epoch, const c10::optional<Tensor>& status,
                     double limit_s) {
  check_cuda(out, "out");
  c10::cuda::CUDAGuard guard(out.device());
  const int* fl = opt_i32(flags);
  bux::ep_pull_combine(u64_ptr(peer_base), rank_of.data_ptr<int>(), row_of.data_ptr<int>(), opt_f32(w), out.data_ptr(),
                       out.size(0), (int)row_of.size(1), (int)out.size(1), fl, fl ? (int)flags->numel() : 0, (int)epoch,
                       (uint64_t)(limit_s * 1e9), status_ptr(status), stream_of(out));
}
void ep_pull_dot(const Tensor& peer_base, const Tensor& rank_of, const Tensor& row_of, const Tensor& dout, Tensor& dw) {
  check_cuda(dout, "dout");
  c10::cuda::CUDAGuard guard(dout.device());
  bux::ep_pull_dot(u64_ptr(peer_base), rank_of.data_ptr<int>(), row_of.data_ptr<int>(), dout.data_ptr(), dw.data_ptr<float>(),
                   row_of.numel(), (int)row_of.size(1), (int)dout.size(1), stream_of(dout));
}
void zero_pad_rows(Tensor& buf, const Tensor& offsets, const Tensor& counts) {
  check_cuda(buf, "buf");
  c10::cuda::CUDAGuard guard(buf.device());
  bux::zero_pad_rows(buf.data_ptr(), offsets.data_ptr<int>(), counts.data_ptr<int>(), (int)counts.numel(), (int)buf.size(-1), stream_of(buf));
}
void tp_push_block(const Tensor& src, const Tensor& peer_base, int64_t my_rank, int64_t sms) {
  check_cuda(src, "src");
  TORCH_CHECK(src.is_contiguous() && src.scalar_type() == at::kBFloat16 && src.size(-1) % 8 == 0, "tp_push_block: contiguous bf16 rows, width % 8 == 0");
  c10::cuda::CUDAGuard guard(src.device());
  const int d = (int)src.size(-1);
  bux::tp_push_block(src.data_ptr(), reinterpret_cast<const uint64_t*>(peer_base.data_ptr<int64_t>()), (int)peer_base.numel(),
                     (int)my_rank, src.numel() / d, d, (int)sms, stream_of(src));
}
void tp_pull_reduce(const Tensor& peer_base, int64_t my_rank, Tensor& out, const c10::optional<Tensor>& residual,
                    const c10::optional<Tensor>& flags, int64_t epoch, const c10::optional<Tensor>& status, double limit_s) {
  check_cuda(out, "out");
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == at::kBFloat16 && out.size(-1) % 8 == 0, "tp_pull_reduce: contiguous bf16 rows");
  c10::cuda::CUDAGuard guard(out.device());
  const int d = (int)out.size(-1);
  bux::tp_pull_reduce(reinterpret_cast<const uint64_t*>(peer_base.data_ptr<int64_t>()), (int)peer_base.numel(), (int)my_rank,
                      out.numel() / d, d, out.data_ptr(), residual.has_value() ? residual->data_ptr() : nullptr,
                      opt_i32(flags), (int)epoch, (uint64_t)(limit_s * 1e9), status_ptr(status), stream_of(out));
}
void set_comm_ctas_per_sm(int64_t n) { bux::set_comm_ctas_per_sm((int)n); }
void sf_rows_to_tiles(const Tensor& src, Tensor& dst) {
  check_cuda(src, "src");
  TORCH_CHECK(src.dim() == 2 && src.scalar_type() == at::kByte && src.is_contiguous() && src.size(1) % 4 == 0 &&
                  dst.scalar_type() == at::kByte && dst.is_contiguous(), "sf_rows_to_tiles: [rows, sf_cols % 4 == 0] bytes");
  const int64_t tiles = ((src.size(0) + 127) / 128) * (src.size(1) / 4) * 512;
  TORCH_CHECK(dst.numel() >= tiles, "sf_rows_to_tiles: the tile buffer holds ", dst.numel(), " bytes, needs ", tiles);
  c10::cuda::CUDAGuard guard(src.device());
  bux::sf_rows_to_tiles(src.data_ptr(), dst.data_ptr(), src.size(0), (int)src.size(1), stream_of(src));
}
void ep_wait(const Tensor& flags, int64_t epoch, const c10::optional<Tensor>& status, double limit_s) {
  c10::cuda::CUDAGuard guard(flags.device());
  bux::ep_wait(flags.data_ptr<int>(), (int)flags.numel(), (int)epoch, (uint64_t)(limit_s * 1e9), status_ptr(status), stream_of(flags));
}

}  // namespace

TORCH_LIBRARY(bux_b200, m) {
  m.def("ep_push_rows(Tensor x, Tensor src_token, Tensor dst_rank, Tensor dst_row, Tensor? row_scale, Tensor peer_base, int sms, Tensor? peer_scale=None) -> ()", &ep_push_rows);
  m.def("ep_push_rows_mx(Tensor x, Tensor rank_of, Tensor row_of, Tensor? w, Tensor peer_q, Tensor peer_sf, Tensor? peer_scale, int sms) -> ()", &ep_push_rows_mx);
  m.def("requant_mxfp8_cols(Tensor q, Tensor sf, Tensor(a!) q_col, Tensor(b!) sf_col, int rows, int cols, int ld_col) -> ()", &requant_mxfp8_cols);
  m.def("row_dots(Tensor a, Tensor b, Tensor(a!) out) -> ()", &row_dots);
  m.def("ep_pull_scalar(Tensor peer_base, Tensor rank_of, Tensor row_of, Tensor(a!) out, Tensor? flags, int epoch, Tensor? status, float limit_s) -> ()", &ep_pull_scalar);
  m.def("ep_signal(Tensor peer_flags, int channel, int world, int my_rank, int epoch) -> ()", &ep_signal);
  m.def("ep_pull_combine(Tensor peer_base, Tensor rank_of, Tensor row_of, Tensor? w, Tensor(a!) out, Tensor? flags, int epoch, Tensor? status, float limit_s) -> ()", &ep_pull_combine);
  m.def("ep_pull_dot(Tensor peer_base, Tensor rank_of, Tensor row_of, Tensor dout, Tensor(a!) dw) -> ()", &ep_pull_dot);
  m.def("zero_pad_rows(Tensor(a!) buf, Tensor offsets, Tensor counts) -> ()", &zero_pad_rows);
  m.def("ep_wait(Tensor flags, int epoch, Tensor? status, float limit_s) -> ()", &ep_wait);
  m.def("set_comm_ctas_per_sm(int n) -> ()", &set_comm_ctas_per_sm);
  m.def("causal_conv(bool bwd, Tensor inp, Tensor w, Tensor? bias, Tensor? position, Tensor(a!) out) -> ()", &causal_conv);
  m.def("causal_conv_wgrad(Tensor x, Tensor dy, Tensor? position, Tensor(a!) dw, Tensor(b!)? db) -> ()", &causal_conv_wgrad);
  m.def("chunk_scan(Tensor a1, Tensor aux1, Tensor? aux3, Tensor a4, Tensor v, Tensor lam, Tensor? s0, Tensor? out, Tensor? x_out, Tensor? states, Tensor(a!) s_last, Tensor? status, int bh, int n_chunks, bool reverse) -> ()", &chunk_scan);
  m.def("sf_rows_to_tiles(Tensor src, Tensor(a!) dst) -> ()", &sf_rows_to_tiles);
  m.def("tp_push_block(Tensor src, Tensor peer_base, int my_rank, int sms) -> ()", &tp_push_block);
  m.def("tp_pull_reduce(Tensor peer_base, int my_rank, Tensor(a!) out, Tensor? residual, Tensor? flags, int epoch, Tensor? status, float limit_s) -> ()", &tp_pull_reduce);
  m.def("gemm(Tensor a, Tensor b, Tensor(a!) c, Tensor? sfa, Tensor? sfb, Tensor? group_offsets, Tensor? status, int kind, int mode, int M, int N, int K, int k_total, int groups, bool a_mn, bool b_mn, int out_kind, int bn, int sms, Tensor? wait_flags=None, int wait_epoch=0, int wait_rows=0, int m_rotate=0, bool wait_on_k=False, bool wait_on_n=False) -> ()", &gemm);
  m.def("rmsnorm_fwd(Tensor x, Tensor? w, Tensor(a!) y, Tensor(b!) rstd, float eps) -> ()", &rmsnorm_fwd);
  m.def("rmsnorm_bwd(Tensor x, Tensor? w, Tensor dy, Tensor rstd, Tensor(a!) dx, Tensor? dw) -> ()", &rmsnorm_bwd);
  m.def("norm_rope(bool bwd, Tensor x, Tensor? w, Tensor cos, Tensor sin, Tensor(a!) y, Tensor? rstd, Tensor? dy, Tensor? dw, int tokens, int heads, int D, int stride_x, int stride_y, float eps) -> ()", &norm_rope);
  m.def("glu_fwd(Tensor h, Tensor(a!) out, Tensor? row_scale, int kind, float limit, float up_offset) -> ()", &glu_fwd);
  m.def("glu_bwd(Tensor h, Tensor dout, Tensor(a!) dh, Tensor? row_scale, Tensor? d_row_scale, int kind, float limit, float up_offset) -> ()", &glu_bwd);
  m.def("quant_mxfp8(Tensor x, Tensor? row_index, Tensor? row_scale, Tensor? q_row, Tensor? sf_row, Tensor? q_col, Tensor? sf_col, int rows, int cols, int ld_col, int batch, int x_batch_stride) -> ()", &quant_mxfp8);
  m.def("quant_mxfp8_glu(Tensor h, Tensor? dout, Tensor? row_scale, Tensor? q_row, Tensor? sf_row, Tensor? q_col, Tensor? sf_col, int ld_col, int kind, float limit, float up_offset) -> ()", &quant_mxfp8_glu);
  m.def("quant_nvfp4(Tensor x, Tensor tensor_scale, Tensor(a!) packed, Tensor(b!) scales) -> ()", &quant_nvfp4);
  m.def("ce_fwd_bwd(Tensor(a!) logits, Tensor targets, Tensor? mask, Tensor(b!) loss, Tensor? logz, float grad_scale, float z_weight, float softcap) -> ()", &ce_fwd_bwd);
  m.def("adamw(Tensor(a!) p, Tensor g, Tensor(b!) m, Tensor(c!) v, Tensor? m_sf, Tensor? v_sf, Tensor? shadow, Tensor? grad_scale, float lr, float b1, float b2, float eps, float wd, float bc1, float bc2, float grad_scale_const) -> ()", &adamw);
  m.def("sumsq(Tensor g, Tensor(a!) out) -> ()", &sumsq);
  m.def("topk_rows(Tensor scores, Tensor(a!) idx) -> ()", &topk_rows);
  m.def("gather_rows(Tensor x, Tensor index, Tensor(a!) out) -> ()", &gather_rows);
  m.def("combine_bwd(Tensor? y, Tensor dout, Tensor pos, Tensor? w, Tensor(a!)? dy, Tensor(b!)? dw) -> ()", &combine_bwd);
  m.def("combine_rows(Tensor y, Tensor pos, Tensor? w, Tensor(a!) out) -> ()", &combine_rows);
  m.def("attn_fwd(Tensor q, Tensor k, Tensor v, Tensor(a!) o, Tensor(b!) lse, Tensor? sinks, Tensor? status, float scale, bool causal, int window, Tensor? row_lo) -> ()", &attn_fwd);
  m.def("attn_bwd(Tensor q, Tensor k, Tensor v, Tensor o, Tensor d_o, Tensor lse, Tensor(a!) dq, Tensor(b!) dk, Tensor(c!) dv, Tensor(d!) delta, Tensor? sinks, Tensor? dsinks, Tensor? status, float scale, bool causal, int window, Tensor? row_lo, Tensor? key_hi, Tensor? phase_cycles=None) -> ()", &attn_bwd);
}
