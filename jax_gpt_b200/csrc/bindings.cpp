// torch bindings for the sm_100a kernels: tensors in, raw pointers + current stream out.
// Registered as torch.ops.b200.* ; no computation happens in this file.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>
#include <torch/torch.h>

#include <cstring>
#include <tuple>
#include <vector>

#include "attention_sm100.cuh"
#include "elementwise.cuh"
#include "gemm_sm100.cuh"

namespace {

using at::Tensor;
using b200::GemmArgs;

#define B200_CHECK_CUDA(expr)                                                              \
  do {                                                                                     \
    cudaError_t _e = (expr);                                                               \
    TORCH_CHECK(_e == cudaSuccess, "b200 kernel launch failed: ", cudaGetErrorString(_e)); \
  } while (0)

const __nv_bfloat16* bf16_ptr(const Tensor& t) { return reinterpret_cast<const __nv_bfloat16*>(t.data_ptr()); }
__nv_bfloat16* bf16_mut(Tensor& t) { return reinterpret_cast<__nv_bfloat16*>(t.data_ptr()); }
const __nv_bfloat16* bf16_opt(const c10::optional<Tensor>& t) {
  return t.has_value() ? reinterpret_cast<const __nv_bfloat16*>(t->data_ptr()) : nullptr;
}
cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_bf16_2d(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16 && t.dim() == 2 && t.stride(1) == 1, name,
              " must be a 2-D bf16 CUDA tensor with unit inner stride");
  TORCH_CHECK(t.stride(0) % 8 == 0 && (reinterpret_cast<uintptr_t>(t.data_ptr()) & 15) == 0, name,
              " must have a 16-byte aligned base and row stride");
}

// One status buffer per device: 4 int32 words written by kernels whose bounded waits expire.
Tensor status_tensor(int device) {
  static std::vector<Tensor> per_device(64);
  if (!per_device[device].defined()) {
    per_device[device] = at::zeros({4}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  }
  return per_device[device];
}
int* status_ptr(const Tensor& like) { return status_tensor(like.get_device()).data_ptr<int>(); }

Tensor status(int64_t device) { return status_tensor(static_cast<int>(device)); }

// out[M,N] = epilogue(alpha * A @ B^T ...). a: [M,K] (or [K,M] if a_mn_major); b: [N,K] (or [K,N]).
void gemm(const Tensor& a, bool a_mn_major, const Tensor& b, bool b_mn_major, Tensor out,
          const c10::optional<Tensor>& bias, const c10::optional<Tensor>& residual, const c10::optional<Tensor>& aux,
          int64_t epilogue, int64_t out_mode, double alpha, int64_t split_k) {
  c10::cuda::CUDAGuard guard(a.device());
  check_bf16_2d(a, "a");
  check_bf16_2d(b, "b");
  const int M = static_cast<int>(a_mn_major ? a.size(1) : a.size(0));
  const int K = static_cast<int>(a_mn_major ? a.size(0) : a.size(1));
  const int N = static_cast<int>(b_mn_major ? b.size(1) : b.size(0));
  const int Kb = static_cast<int>(b_mn_major ? b.size(0) : b.size(1));
  TORCH_CHECK(K == Kb, "gemm: contraction sizes differ: ", K, " vs ", Kb);
  TORCH_CHECK(out.is_cuda() && out.dim() == 2 && out.size(0) == M && out.size(1) == N && out.stride(1) == 1,
              "gemm: out must be [M,N] with unit inner stride");
  GemmArgs g{};
  g.M = M;
  g.N = N;
  g.K = K;
  g.out = out.data_ptr();
  g.ldo = out.stride(0);
  g.out_mode = static_cast<int>(out_mode);
  if (g.out_mode == b200::kOutBf16) {
    TORCH_CHECK(out.scalar_type() == at::kBFloat16, "gemm: out must be bf16");
  } else {
    TORCH_CHECK(out.scalar_type() == at::kFloat, "gemm: out must be fp32 for this output mode");
  }
  g.bias = bf16_opt(bias);
  if (bias.has_value()) {
    TORCH_CHECK(bias->numel() == N && bias->scalar_type() == at::kBFloat16, "gemm: bad bias");
  }
  g.residual = bf16_opt(residual);
  g.ldr = residual.has_value() ? residual->stride(0) : 0;
  if (residual.has_value()) {
    TORCH_CHECK(residual->scalar_type() == at::kBFloat16 && residual->size(0) == M && residual->size(1) == N,
                "gemm: bad residual");
  }
  g.epilogue = static_cast<int>(epilogue);
  if (g.epilogue == b200::kEpiGelu) {
    TORCH_CHECK(aux.has_value() && aux->scalar_type() == at::kBFloat16 && aux->size(0) == M && aux->size(1) == N,
                "gemm: GELU epilogue needs an [M,N] bf16 aux output");
    g.aux_out = reinterpret_cast<__nv_bfloat16*>(aux->data_ptr());
    g.ldaux = aux->stride(0);
  } else if (g.epilogue == b200::kEpiGeluGrad) {
    TORCH_CHECK(aux.has_value() && aux->scalar_type() == at::kBFloat16 && aux->size(0) == M && aux->size(1) == N,
                "gemm: GELU-grad epilogue needs the [M,N] bf16 pre-activation");
    g.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux->data_ptr());
    g.ldaux = aux->stride(0);
  }
  g.alpha = static_cast<float>(alpha);
  g.split_k = static_cast<int>(split_k);
  g.status = status_ptr(a);
  B200_CHECK_CUDA(b200::launch_gemm_bf16(bf16_ptr(a), a.stride(0), a_mn_major ? 1 : 0, bf16_ptr(b), b.stride(0),
                                         b_mn_major ? 1 : 0, g, cur_stream()));
}

// All-gather -> GEMM, the gather pushed by copier CTAs of the same kernel. gather_ptrs[s] / ready_ptrs[s]: rank s's
// gather buffer [n * rows_per_src, K] bf16 and ready array int32[n * rows_per_src / 128] as mapped here (entry `rank`
// = this rank's own, whose block `rank` already holds the local rows).
void gemm_gathered_a_staged(std::vector<int64_t> gather_ptrs, std::vector<int64_t> ready_ptrs, int64_t rows_per_src,
                            int64_t K, int64_t rank, const Tensor& b, bool b_mn_major, Tensor out,
                            const c10::optional<Tensor>& bias, int64_t epoch, double wait_seconds) {
  c10::cuda::CUDAGuard guard(b.device());
  check_bf16_2d(b, "b");
  const int n = static_cast<int>(gather_ptrs.size());
  TORCH_CHECK(n >= 1 && n <= b200::kMaxPeers && ready_ptrs.size() == gather_ptrs.size() && rank >= 0 && rank < n,
              "gemm_gathered_a_staged: 1..8 ranks");
  GemmArgs g{};
  g.M = static_cast<int>(rows_per_src * n);
  g.K = static_cast<int>(K);
  g.N = static_cast<int>(b_mn_major ? b.size(1) : b.size(0));
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.size(0) == g.M && out.size(1) == g.N, "gemm_gathered_a_staged: bad out");
  g.out = out.data_ptr();
  g.ldo = out.stride(0);
  g.out_mode = b200::kOutBf16;
  g.bias = bf16_opt(bias);
  g.alpha = 1.f;
  g.split_k = 1;
  g.status = status_ptr(b);
  __nv_bfloat16* peers[b200::kMaxPeers];
  int* ready[b200::kMaxPeers];
  for (int i = 0; i < n; ++i) {
    peers[i] = reinterpret_cast<__nv_bfloat16*>(gather_ptrs[i]);
    ready[i] = reinterpret_cast<int*>(ready_ptrs[i]);
  }
  B200_CHECK_CUDA(b200::launch_gemm_bf16_gathered_a_staged(peers, ready, n, static_cast<int>(rows_per_src),
                                                           static_cast<int>(rank), bf16_ptr(b), b.stride(0),
                                                           b_mn_major ? 1 : 0, g, static_cast<int>(epoch), wait_seconds,
                                                           cur_stream()));
}

// x [M, K] @ W [K, N], W column-sharded over the ranks and pushed into every rank's gather buffer by copier CTAs of
// the same kernel. w_ptrs[s] / ready_ptrs[s]: rank s's buffer (n matrices [K, N / n] bf16) and ready array
// int32[n * K / 64] as mapped here.
void gemm_sharded_b_staged(const Tensor& a, std::vector<int64_t> w_ptrs, std::vector<int64_t> ready_ptrs, int64_t N,
                           int64_t rank, Tensor out, const c10::optional<Tensor>& bias, int64_t epoch, double wait_seconds) {
  c10::cuda::CUDAGuard guard(a.device());
  check_bf16_2d(a, "a");
  const int n = static_cast<int>(w_ptrs.size());
  TORCH_CHECK(n >= 1 && n <= b200::kMaxPeers && ready_ptrs.size() == w_ptrs.size() && rank >= 0 && rank < n,
              "gemm_sharded_b_staged: 1..8 ranks");
  GemmArgs g{};
  g.M = static_cast<int>(a.size(0));
  g.K = static_cast<int>(a.size(1));
  g.N = static_cast<int>(N);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.size(0) == g.M && out.size(1) == g.N, "gemm_sharded_b_staged: bad out");
  g.out = out.data_ptr();
  g.ldo = out.stride(0);
  g.out_mode = b200::kOutBf16;
  g.bias = bf16_opt(bias);
  g.alpha = 1.f;
  g.split_k = 1;
  g.status = status_ptr(a);
  __nv_bfloat16* peers[b200::kMaxPeers];
  int* ready[b200::kMaxPeers];
  for (int i = 0; i < n; ++i) {
    peers[i] = reinterpret_cast<__nv_bfloat16*>(w_ptrs[i]);
    ready[i] = reinterpret_cast<int*>(ready_ptrs[i]);
  }
  B200_CHECK_CUDA(b200::launch_gemm_bf16_sharded_b_staged(bf16_ptr(a), a.stride(0), peers, ready, n, static_cast<int>(rank),
                                                          g, static_cast<int>(epoch), wait_seconds, cur_stream()));
}

// GEMM -> reduce-scatter, partial tiles pushed to the row owners and summed there (one kernel).
// recv_ptrs[r] / cnt_ptrs[r]: rank r's receive buffer [n, rows_per_peer, N] bf16 and arrival counters as mapped here.
void gemm_reduce_scatter_push(const Tensor& a, const Tensor& b, bool b_mn_major, std::vector<int64_t> recv_ptrs,
                              std::vector<int64_t> cnt_ptrs, int64_t rank, int64_t rows_per_peer, Tensor out,
                              int64_t cnt_expected, double wait_seconds) {
  c10::cuda::CUDAGuard guard(a.device());
  check_bf16_2d(a, "a");
  check_bf16_2d(b, "b");
  const int n = static_cast<int>(recv_ptrs.size());
  TORCH_CHECK(n >= 1 && n <= b200::kMaxPeers && cnt_ptrs.size() == recv_ptrs.size() && rank >= 0 && rank < n,
              "gemm_reduce_scatter_push: 1..8 peers");
  GemmArgs g{};
  g.M = static_cast<int>(a.size(0));
  g.K = static_cast<int>(a.size(1));
  g.N = static_cast<int>(b_mn_major ? b.size(1) : b.size(0));
  TORCH_CHECK(rows_per_peer * n == g.M && rows_per_peer % 128 == 0 && g.N % 64 == 0,
              "gemm_reduce_scatter_push: M = peers * rows_per_peer, rows_per_peer % 128 == 0, N % 64 == 0");
  TORCH_CHECK(out.is_contiguous() && out.scalar_type() == at::kBFloat16 && out.size(0) == rows_per_peer && out.size(1) == g.N,
              "gemm_reduce_scatter_push: out [rows_per_peer, N] bf16");
  g.out = nullptr;
  g.ldo = g.N;
  g.out_mode = b200::kOutBf16PeerPush;
  g.n_peers = n;
  g.self_rank = static_cast<int>(rank);
  g.rows_per_peer = static_cast<int>(rows_per_peer);
  for (int i = 0; i < n; ++i) {
    g.peer_out[i] = reinterpret_cast<float*>(recv_ptrs[i]);
    g.peer_cnt[i] = reinterpret_cast<int*>(cnt_ptrs[i]);
  }
  g.cnt_expected = static_cast<int>(cnt_expected);
  g.rs_out = bf16_mut(out);
  g.rs_wait_ns = static_cast<unsigned long long>((wait_seconds > 0 ? wait_seconds : 20.0) * 1e9);
  g.alpha = 1.f;
  g.split_k = 1;
  g.status = status_ptr(a);
  B200_CHECK_CUDA(b200::launch_gemm_bf16_reduce_scatter_push(bf16_ptr(a), a.stride(0), bf16_ptr(b), b.stride(0),
                                                             b_mn_major ? 1 : 0, g, cur_stream()));
}

void norm_fwd(int64_t mode, const Tensor& x, const Tensor& gamma, const c10::optional<Tensor>& beta, Tensor y,
              c10::optional<Tensor> mean, c10::optional<Tensor> rstd, double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && x.scalar_type() == at::kBFloat16, "norm_fwd: contiguous bf16");
  const int D = static_cast<int>(x.size(-1));
  const int M = static_cast<int>(x.numel() / D);
  B200_CHECK_CUDA(b200::launch_norm_fwd(static_cast<int>(mode), bf16_ptr(x), bf16_ptr(gamma), bf16_opt(beta),
                                        bf16_mut(y), mean.has_value() ? mean->data_ptr<float>() : nullptr,
                                        rstd.has_value() ? rstd->data_ptr<float>() : nullptr, M, D,
                                        static_cast<float>(eps), cur_stream()));
}

void norm_bwd(int64_t mode, const Tensor& dy, const Tensor& x, const Tensor& gamma, const c10::optional<Tensor>& mean,
              const Tensor& rstd, const c10::optional<Tensor>& dres, Tensor dx, Tensor dgamma,
              c10::optional<Tensor> dbeta, Tensor scratch) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && dx.is_contiguous(), "norm_bwd: contiguous tensors");
  TORCH_CHECK(dgamma.scalar_type() == at::kFloat, "norm_bwd: dgamma must be fp32");
  const int D = static_cast<int>(x.size(-1));
  TORCH_CHECK(scratch.scalar_type() == at::kFloat && scratch.is_contiguous() &&
                  scratch.numel() >= b200::norm_bwd_scratch_floats(D),
              "norm_bwd: scratch must hold ", b200::norm_bwd_scratch_floats(D), " floats");
  const int M = static_cast<int>(x.numel() / D);
  B200_CHECK_CUDA(b200::launch_norm_bwd(static_cast<int>(mode), bf16_ptr(dy), bf16_ptr(x), bf16_ptr(gamma),
                                        mean.has_value() ? mean->data_ptr<float>() : nullptr, rstd.data_ptr<float>(),
                                        bf16_opt(dres), bf16_mut(dx), dgamma.data_ptr<float>(),
                                        dbeta.has_value() ? dbeta->data_ptr<float>() : nullptr,
                                        scratch.data_ptr<float>(), M, D, cur_stream()));
}

void embed_fwd(const Tensor& idx, const Tensor& wte, const c10::optional<Tensor>& wpe, Tensor out, int64_t T,
               int64_t pos0) {
  c10::cuda::CUDAGuard guard(idx.device());
  TORCH_CHECK(idx.scalar_type() == at::kInt && idx.is_contiguous(), "embed_fwd: int32 contiguous indices");
  const int D = static_cast<int>(wte.size(1));
  B200_CHECK_CUDA(b200::launch_embed_fwd(idx.data_ptr<int>(), bf16_ptr(wte), bf16_opt(wpe), bf16_mut(out),
                                         static_cast<int>(idx.numel()), static_cast<int>(T), D,
                                         static_cast<int>(pos0), cur_stream()));
}

void embed_bwd(const Tensor& idx, const Tensor& dout, Tensor dwte, c10::optional<Tensor> dwpe, int64_t T,
               int64_t pos0) {
  c10::cuda::CUDAGuard guard(idx.device());
  TORCH_CHECK(dwte.scalar_type() == at::kFloat, "embed_bwd: fp32 gradient buffers");
  const int D = static_cast<int>(dwte.size(1));
  B200_CHECK_CUDA(b200::launch_embed_bwd(idx.data_ptr<int>(), bf16_ptr(dout), dwte.data_ptr<float>(),
                                         dwpe.has_value() ? dwpe->data_ptr<float>() : nullptr,
                                         static_cast<int>(idx.numel()), static_cast<int>(T), D,
                                         static_cast<int>(pos0), cur_stream()));
}

void ce_fwd_bwd(Tensor logits, const Tensor& targets, Tensor loss, int64_t V, double scale, bool write_grad) {
  c10::cuda::CUDAGuard guard(logits.device());
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1 && logits.scalar_type() == at::kBFloat16, "ce: bf16 logits");
  TORCH_CHECK(targets.scalar_type() == at::kInt && loss.scalar_type() == at::kFloat, "ce: int32 targets, fp32 loss");
  B200_CHECK_CUDA(b200::launch_ce_fwd_bwd(bf16_mut(logits), targets.data_ptr<int>(), loss.data_ptr<float>(),
                                          static_cast<int>(logits.size(0)), static_cast<int>(V),
                                          static_cast<int>(logits.stride(0)), static_cast<float>(scale),
                                          write_grad ? 1 : 0, cur_stream()));
}

void bias_grad(const Tensor& dy, Tensor dbias) {
  c10::cuda::CUDAGuard guard(dy.device());
  TORCH_CHECK(dy.is_contiguous() && dy.dim() == 2 && dbias.scalar_type() == at::kFloat, "bias_grad: bad arguments");
  B200_CHECK_CUDA(b200::launch_bias_grad(bf16_ptr(dy), dbias.data_ptr<float>(), static_cast<int>(dy.size(0)),
                                         static_cast<int>(dy.size(1)), cur_stream()));
}

void sumsq(const Tensor& g, Tensor out) {
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.is_contiguous() && g.scalar_type() == at::kFloat && out.scalar_type() == at::kFloat, "sumsq: fp32");
  B200_CHECK_CUDA(b200::launch_sumsq(g.data_ptr<float>(), g.numel(), out.data_ptr<float>(), cur_stream()));
}

void adamw(Tensor p, Tensor g, Tensor m, Tensor v, c10::optional<Tensor> p_bf16, const Tensor& hp,
           const c10::optional<Tensor>& gnorm_sq, double beta1, double beta2, double eps, double wd, double clip,
           bool zero_grad) {
  c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw: contiguous");
  TORCH_CHECK(p.scalar_type() == at::kFloat && g.scalar_type() == at::kFloat, "adamw: fp32 master and grad");
  B200_CHECK_CUDA(b200::launch_adamw(
      p.data_ptr<float>(), g.data_ptr<float>(), m.data_ptr<float>(), v.data_ptr<float>(),
      p_bf16.has_value() ? reinterpret_cast<__nv_bfloat16*>(p_bf16->data_ptr()) : nullptr, p.numel(),
      hp.data_ptr<float>(), gnorm_sq.has_value() ? gnorm_sq->data_ptr<float>() : nullptr, static_cast<float>(beta1),
      static_cast<float>(beta2), static_cast<float>(eps), static_cast<float>(wd), static_cast<float>(clip),
      zero_grad ? 1 : 0, cur_stream()));
}

void adamw_bf16_state(Tensor p, Tensor g, Tensor m, Tensor v, const Tensor& hp, const c10::optional<Tensor>& gnorm_sq,
                      double beta1, double beta2, double eps, double wd, double clip, bool zero_grad, int64_t seed) {
  c10::cuda::CUDAGuard guard(p.device());
  TORCH_CHECK(p.numel() == g.numel() && p.numel() == m.numel() && p.numel() == v.numel(), "adamw_bf16_state: sizes differ");
  TORCH_CHECK(p.is_contiguous() && g.is_contiguous() && m.is_contiguous() && v.is_contiguous(), "adamw_bf16_state: contiguous");
  TORCH_CHECK(p.scalar_type() == at::kBFloat16 && m.scalar_type() == at::kBFloat16 && v.scalar_type() == at::kBFloat16 &&
                  g.scalar_type() == at::kFloat,
              "adamw_bf16_state: bf16 weights and moments, fp32 gradient");
  B200_CHECK_CUDA(b200::launch_adamw_bf16_state(
      bf16_mut(p), g.data_ptr<float>(), bf16_mut(m), bf16_mut(v), p.numel(), hp.data_ptr<float>(),
      gnorm_sq.has_value() ? gnorm_sq->data_ptr<float>() : nullptr, static_cast<float>(beta1), static_cast<float>(beta2),
      static_cast<float>(eps), static_cast<float>(wd), static_cast<float>(clip), zero_grad ? 1 : 0,
      static_cast<uint32_t>(seed), cur_stream()));
}

// q/k/v: 2-D bf16 views [B*T, H*D] (possibly column slices of one fused buffer).
void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor out, Tensor lse, int64_t B, int64_t T,
              int64_t H, int64_t Hkv, int64_t D, double scale, bool causal, int64_t Dv) {
  c10::cuda::CUDAGuard guard(q.device());
  check_bf16_2d(q, "q");
  check_bf16_2d(k, "k");
  check_bf16_2d(v, "v");
  check_bf16_2d(out, "out");
  b200::AttnTensors t{bf16_ptr(q), bf16_ptr(k), bf16_ptr(v), q.stride(0), k.stride(0), v.stride(0)};
  b200::AttnShape s{static_cast<int>(B), static_cast<int>(T), static_cast<int>(H), static_cast<int>(Hkv),
                    static_cast<int>(D), static_cast<float>(scale), causal ? 1 : 0, static_cast<int>(Dv)};
  B200_CHECK_CUDA(b200::launch_attn_fwd(t, s, bf16_mut(out), out.stride(0), lse.data_ptr<float>(), status_ptr(q),
                                        cur_stream()));
}

void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& dout,
              const Tensor& lse, Tensor delta, Tensor dq_accum, Tensor dk, Tensor dv, int64_t B, int64_t T, int64_t H,
              int64_t Hkv, int64_t D, double scale, bool causal) {
  c10::cuda::CUDAGuard guard(q.device());
  check_bf16_2d(q, "q");
  check_bf16_2d(k, "k");
  check_bf16_2d(v, "v");
  check_bf16_2d(out, "out");
  check_bf16_2d(dout, "dout");
  check_bf16_2d(dk, "dk");
  check_bf16_2d(dv, "dv");
  TORCH_CHECK(dq_accum.scalar_type() == at::kFloat && dq_accum.is_contiguous(), "attn_bwd: dq_accum fp32 contiguous");
  b200::AttnTensors t{bf16_ptr(q), bf16_ptr(k), bf16_ptr(v), q.stride(0), k.stride(0), v.stride(0)};
  b200::AttnShape s{static_cast<int>(B), static_cast<int>(T), static_cast<int>(H), static_cast<int>(Hkv),
                    static_cast<int>(D), static_cast<float>(scale), causal ? 1 : 0, 0};
  B200_CHECK_CUDA(b200::launch_attn_bwd(t, s, bf16_ptr(out), out.stride(0), bf16_ptr(dout), dout.stride(0),
                                        lse.data_ptr<float>(), delta.data_ptr<float>(), dq_accum.data_ptr<float>(),
                                        bf16_mut(dk), dk.stride(0), bf16_mut(dv), dv.stride(0), status_ptr(q),
                                        cur_stream()));
}

// Forward with keys / values read from a cache (B, Hkv, max_len, D) and queries at positions q_pos0 + i.
// q, out: 2-D views [B*Tq, H*D]; kcache, vcache: 4-D bf16 with contiguous rows of D (Dv) elements.
void attn_fwd_cached(const Tensor& q, const Tensor& kcache, const Tensor& vcache, Tensor out, Tensor lse, int64_t B,
                     int64_t Tq, int64_t H, int64_t Tk, int64_t q_pos0, double scale, bool causal) {
  c10::cuda::CUDAGuard guard(q.device());
  check_bf16_2d(q, "q");
  check_bf16_2d(out, "out");
  TORCH_CHECK(kcache.dim() == 4 && vcache.dim() == 4 && kcache.scalar_type() == at::kBFloat16 &&
                  vcache.scalar_type() == at::kBFloat16 && kcache.is_contiguous() && vcache.is_contiguous(),
              "attn_fwd_cached: caches must be contiguous bf16 (B, Hkv, max_len, D)");
  const int64_t Hkv = kcache.size(1), max_len = kcache.size(2), D = kcache.size(3), Dv = vcache.size(3);
  TORCH_CHECK(kcache.size(0) >= B && vcache.size(0) == kcache.size(0) && vcache.size(1) == Hkv &&
                  vcache.size(2) == max_len && Tk <= max_len && q_pos0 >= 0,
              "attn_fwd_cached: cache shape");
  b200::AttnTensors t{bf16_ptr(q), bf16_ptr(kcache), bf16_ptr(vcache), q.stride(0), D, Dv};
  b200::AttnShape s{static_cast<int>(B), static_cast<int>(Tq), static_cast<int>(H), static_cast<int>(Hkv),
                    static_cast<int>(D), static_cast<float>(scale), causal ? 1 : 0, static_cast<int>(Dv)};
  b200::AttnKvLayout kv;
  kv.Tk = static_cast<int>(Tk);
  kv.q_pos0 = static_cast<int>(q_pos0);
  kv.rows_b = static_cast<int>(Hkv * max_len);
  kv.rows_h = static_cast<int>(max_len);
  kv.k_col_h = 0;
  kv.v_col_h = 0;
  kv.rows = static_cast<uint64_t>(kcache.size(0) * Hkv * max_len);
  kv.k_cols = static_cast<uint64_t>(D);
  kv.v_cols = static_cast<uint64_t>(Dv);
  B200_CHECK_CUDA(b200::launch_attn_fwd_kv(t, s, kv, bf16_mut(out), out.stride(0), lse.data_ptr<float>(),
                                           status_ptr(q), cur_stream()));
}

// Gradients for the wide heads: (D, Dv) = (256, 256) or (192, 128).
void attn_bwd_wide(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& out, const Tensor& dout,
                   const Tensor& lse, Tensor delta, Tensor dq_accum, Tensor dk, Tensor dv, int64_t B, int64_t T,
                   int64_t H, int64_t Hkv, int64_t D, int64_t Dv, double scale, bool causal) {
  c10::cuda::CUDAGuard guard(q.device());
  check_bf16_2d(q, "q");
  check_bf16_2d(k, "k");
  check_bf16_2d(v, "v");
  check_bf16_2d(out, "out");
  check_bf16_2d(dout, "dout");
  check_bf16_2d(dk, "dk");
  check_bf16_2d(dv, "dv");
  TORCH_CHECK(dq_accum.scalar_type() == at::kFloat && dq_accum.is_contiguous() && dq_accum.numel() == B * T * H * D,
              "attn_bwd_wide: dq_accum fp32 contiguous [B*T, H*D]");
  TORCH_CHECK(delta.scalar_type() == at::kFloat && delta.numel() == B * H * T && lse.scalar_type() == at::kFloat &&
                  lse.numel() == B * H * T,
              "attn_bwd_wide: lse / delta fp32 [B, H, T]");
  b200::AttnTensors t{bf16_ptr(q), bf16_ptr(k), bf16_ptr(v), q.stride(0), k.stride(0), v.stride(0)};
  b200::AttnShape s{static_cast<int>(B), static_cast<int>(T), static_cast<int>(H), static_cast<int>(Hkv),
                    static_cast<int>(D), static_cast<float>(scale), causal ? 1 : 0, static_cast<int>(Dv)};
  B200_CHECK_CUDA(b200::launch_attn_delta(bf16_ptr(out), out.stride(0), bf16_ptr(dout), dout.stride(0),
                                          delta.data_ptr<float>(), s.B, s.T, s.H, s.Dv, cur_stream()));
  B200_CHECK_CUDA(b200::launch_attn_bwd_wide(t, s, bf16_ptr(dout), dout.stride(0), lse.data_ptr<float>(),
                                             delta.data_ptr<float>(), dq_accum.data_ptr<float>(), bf16_mut(dk),
                                             dk.stride(0), bf16_mut(dv), dv.stride(0), status_ptr(q), cur_stream()));
}

// One query token per sequence against a dense cache. q, out: [B, H*D]; caches (B', Hkv, max_len, D) bf16 with
// unit inner stride; pos: optional int32 device scalar (valid keys = pos + len_add), else `len` keys.
void attn_decode(const Tensor& q, const Tensor& kcache, const Tensor& vcache, const c10::optional<Tensor>& pos,
                 int64_t len, int64_t len_add, int64_t H, double scale, Tensor part_o, Tensor part_ml, Tensor out) {
  c10::cuda::CUDAGuard guard(q.device());
  check_bf16_2d(q, "q");
  check_bf16_2d(out, "out");
  TORCH_CHECK(kcache.dim() == 4 && kcache.scalar_type() == at::kBFloat16 && kcache.stride(3) == 1 &&
                  vcache.scalar_type() == at::kBFloat16 && vcache.sizes() == kcache.sizes() &&
                  vcache.strides() == kcache.strides(),
              "attn_decode: caches must be bf16 (B, Hkv, max_len, D) with equal strides and unit inner stride");
  const int64_t B = q.size(0), Hkv = kcache.size(1), D = kcache.size(3);
  TORCH_CHECK(q.size(1) == H * D && out.size(0) == B && out.size(1) == H * D && kcache.size(0) >= B,
              "attn_decode: q / out must be [B, H*D]");
  TORCH_CHECK(part_o.scalar_type() == at::kFloat && part_ml.scalar_type() == at::kFloat && part_o.is_contiguous() &&
                  part_ml.is_contiguous() && part_o.dim() == 4 && part_o.size(0) >= B && part_o.size(1) == H &&
                  part_o.size(3) == D && part_ml.numel() * D == part_o.numel() * 2,
              "attn_decode: part_o [B, H, splits, D], part_ml [B, H, splits, 2] fp32");
  const int n_splits = static_cast<int>(part_o.size(2));
  const int* pp = nullptr;
  if (pos.has_value()) {
    TORCH_CHECK(pos->scalar_type() == at::kInt && pos->is_cuda(), "attn_decode: pos must be an int32 device tensor");
    pp = pos->data_ptr<int>();
  } else {
    TORCH_CHECK(len <= kcache.size(2), "attn_decode: len exceeds the cache");
  }
  B200_CHECK_CUDA(b200::launch_attn_decode(bf16_ptr(q), q.stride(0), bf16_ptr(kcache), bf16_ptr(vcache),
                                           kcache.stride(0), kcache.stride(1), kcache.stride(2), pp,
                                           static_cast<int>(len), static_cast<int>(len_add), static_cast<int>(B),
                                           static_cast<int>(H), static_cast<int>(Hkv), static_cast<int>(D),
                                           static_cast<float>(scale), n_splits, part_o.data_ptr<float>(),
                                           part_ml.data_ptr<float>(), bf16_mut(out), out.stride(0), cur_stream()));
}

// One query token per sequence against a paged cache: pool [n_pages, page_size, 2 * Hkv * D] bf16 (K of every kv head,
// then V), block_table [max_seqs, max_pages] / seq_ids [B] / seq_lens [max_seqs] int32 on the device.
void attn_decode_paged(const Tensor& q, const Tensor& pool, const Tensor& block_table, const Tensor& seq_ids,
                       const Tensor& seq_lens, int64_t len_add, int64_t H, int64_t Hkv, double scale, Tensor part_o,
                       Tensor part_ml, Tensor out) {
  c10::cuda::CUDAGuard guard(q.device());
  check_bf16_2d(q, "q");
  check_bf16_2d(out, "out");
  TORCH_CHECK(pool.dim() == 3 && pool.is_contiguous() && pool.scalar_type() == at::kBFloat16 && Hkv >= 1 &&
                  pool.size(2) % (2 * Hkv) == 0,
              "attn_decode_paged: pool [n_pages, page_size, 2 * Hkv * D] bf16");
  const int64_t B = q.size(0), D = pool.size(2) / (2 * Hkv);
  auto i32 = [](const Tensor& t) { return t.is_cuda() && t.scalar_type() == at::kInt && t.is_contiguous(); };
  TORCH_CHECK(i32(block_table) && block_table.dim() == 2 && i32(seq_ids) && seq_ids.numel() >= B && i32(seq_lens) &&
                  seq_lens.numel() == block_table.size(0),
              "attn_decode_paged: block_table [max_seqs, max_pages], seq_ids [B], seq_lens [max_seqs] int32 on the device");
  TORCH_CHECK(q.size(1) == H * D && out.size(0) == B && out.size(1) == H * D, "attn_decode_paged: q / out must be [B, H*D]");
  TORCH_CHECK(part_o.scalar_type() == at::kFloat && part_ml.scalar_type() == at::kFloat && part_o.is_contiguous() &&
                  part_ml.is_contiguous() && part_o.dim() == 4 && part_o.size(0) >= B && part_o.size(1) == H &&
                  part_o.size(3) == D && part_ml.numel() * D == part_o.numel() * 2,
              "attn_decode_paged: part_o [B, H, splits, D], part_ml [B, H, splits, 2] fp32");
  B200_CHECK_CUDA(b200::launch_attn_decode_paged(
      bf16_ptr(q), q.stride(0), bf16_ptr(pool), static_cast<int>(pool.size(2)), block_table.data_ptr<int>(),
      seq_ids.data_ptr<int>(), seq_lens.data_ptr<int>(), static_cast<int>(len_add), static_cast<int>(pool.size(1)),
      static_cast<int>(block_table.size(1)), static_cast<int>(B), static_cast<int>(H), static_cast<int>(Hkv),
      static_cast<int>(D), static_cast<float>(scale), static_cast<int>(part_o.size(2)), part_o.data_ptr<float>(),
      part_ml.data_ptr<float>(), bf16_mut(out), out.stride(0), cur_stream()));
}

void attn_bwd_probs(Tensor s, Tensor dp, const Tensor& lse, const Tensor& delta, int64_t c, int64_t q0, double scale,
                    bool causal) {
  c10::cuda::CUDAGuard guard(s.device());
  TORCH_CHECK(s.is_cuda() && s.is_contiguous() && dp.is_contiguous() && s.scalar_type() == at::kBFloat16 &&
                  dp.scalar_type() == at::kBFloat16 && s.sizes() == dp.sizes() && s.dim() >= 2,
              "attn_bwd_probs: s, dp [..., kv] contiguous bf16 of one shape");
  const int64_t kv = s.size(-1), rows = s.numel() / kv;
  TORCH_CHECK(kv % 8 == 0 && lse.is_contiguous() && delta.is_contiguous() && lse.scalar_type() == at::kFloat &&
                  delta.scalar_type() == at::kFloat && lse.numel() == rows && delta.numel() == rows,
              "attn_bwd_probs: kv multiple of 8; lse, delta fp32 with one value per row");
  B200_CHECK_CUDA(b200::launch_attn_bwd_probs(bf16_mut(s), bf16_mut(dp), lse.data_ptr<float>(), delta.data_ptr<float>(),
                                              rows, static_cast<int>(kv), static_cast<int>(c), static_cast<int>(q0),
                                              static_cast<float>(scale), causal ? 1 : 0, cur_stream()));
}

void cast_rows(const Tensor& src, Tensor dst) {
  c10::cuda::CUDAGuard guard(src.device());
  TORCH_CHECK(src.dim() == 2 && dst.dim() == 2 && src.stride(1) == 1 && dst.stride(1) == 1, "cast_rows: 2-D");
  TORCH_CHECK(src.scalar_type() == at::kFloat && dst.scalar_type() == at::kBFloat16, "cast_rows: fp32 -> bf16");
  B200_CHECK_CUDA(b200::launch_cast_rows_f32_bf16(src.data_ptr<float>(), src.stride(0), bf16_mut(dst), dst.stride(0),
                                                  static_cast<int>(src.size(0)), static_cast<int>(src.size(1)),
                                                  cur_stream()));
}

}  // namespace

#include "bindings_extra.inc"

void b200_register_runtime(torch::Library& m);

TORCH_LIBRARY(b200, m) {
  m.def("status(int device) -> Tensor", &status);
  m.def(
      "gemm(Tensor a, bool a_mn_major, Tensor b, bool b_mn_major, Tensor(a!) out, Tensor? bias, Tensor? residual, "
      "Tensor? aux, int epilogue, int out_mode, float alpha, int split_k) -> ()",
      &gemm);
  m.def(
      "gemm_gathered_a_staged(int[] gather_ptrs, int[] ready_ptrs, int rows_per_src, int K, int rank, Tensor b, "
      "bool b_mn_major, Tensor(a!) out, Tensor? bias, int epoch, float wait_seconds) -> ()",
      &gemm_gathered_a_staged);
  m.def(
      "gemm_sharded_b_staged(Tensor a, int[] w_ptrs, int[] ready_ptrs, int N, int rank, Tensor(a!) out, Tensor? bias, "
      "int epoch, float wait_seconds) -> ()",
      &gemm_sharded_b_staged);
  m.def(
      "gemm_reduce_scatter_push(Tensor a, Tensor b, bool b_mn_major, int[] recv_ptrs, int[] cnt_ptrs, int rank, "
      "int rows_per_peer, Tensor(a!) out, int cnt_expected, float wait_seconds) -> ()",
      &gemm_reduce_scatter_push);
  m.def(
      "norm_fwd(int mode, Tensor x, Tensor gamma, Tensor? beta, Tensor(a!) y, Tensor(b!)? mean, Tensor(c!)? rstd, "
      "float eps) -> ()",
      &norm_fwd);
  m.def(
      "norm_bwd(int mode, Tensor dy, Tensor x, Tensor gamma, Tensor? mean, Tensor rstd, Tensor? dres, Tensor(a!) dx, "
      "Tensor(b!) dgamma, Tensor(c!)? dbeta, Tensor(d!) scratch) -> ()",
      &norm_bwd);
  m.def("embed_fwd(Tensor idx, Tensor wte, Tensor? wpe, Tensor(a!) out, int T, int pos0) -> ()", &embed_fwd);
  m.def("embed_bwd(Tensor idx, Tensor dout, Tensor(a!) dwte, Tensor(b!)? dwpe, int T, int pos0) -> ()", &embed_bwd);
  m.def("ce_fwd_bwd(Tensor(a!) logits, Tensor targets, Tensor(b!) loss, int V, float scale, bool write_grad) -> ()",
        &ce_fwd_bwd);
  m.def("bias_grad(Tensor dy, Tensor(a!) dbias) -> ()", &bias_grad);
  m.def("sumsq(Tensor g, Tensor(a!) out) -> ()", &sumsq);
  m.def(
      "adamw(Tensor(a!) p, Tensor(b!) g, Tensor(c!) m, Tensor(d!) v, Tensor(e!)? p_bf16, Tensor hp, Tensor? gnorm_sq, "
      "float beta1, float beta2, float eps, float wd, float clip, bool zero_grad) -> ()",
      &adamw);
  m.def(
      "attn_fwd(Tensor q, Tensor k, Tensor v, Tensor(a!) out, Tensor(b!) lse, int B, int T, int H, int Hkv, int D, "
      "float scale, bool causal, int Dv) -> ()",
      &attn_fwd);
  m.def(
      "attn_bwd(Tensor q, Tensor k, Tensor v, Tensor out, Tensor dout, Tensor lse, Tensor(a!) delta, Tensor(b!) "
      "dq_accum, Tensor(c!) dk, Tensor(d!) dv, int B, int T, int H, int Hkv, int D, float scale, bool causal) -> ()",
      &attn_bwd);
  m.def("cast_rows(Tensor src, Tensor(a!) dst) -> ()", &cast_rows);
  m.def(
      "adamw_bf16_state(Tensor(a!) p, Tensor(b!) g, Tensor(c!) m, Tensor(d!) v, Tensor hp, Tensor? gnorm_sq, float beta1, "
      "float beta2, float eps, float wd, float clip, bool zero_grad, int seed) -> ()",
      &adamw_bf16_state);
  m.def(
      "attn_fwd_cached(Tensor q, Tensor kcache, Tensor vcache, Tensor(a!) out, Tensor(b!) lse, int B, int Tq, int H, "
      "int Tk, int q_pos0, float scale, bool causal) -> ()",
      &attn_fwd_cached);
  m.def(
      "attn_bwd_wide(Tensor q, Tensor k, Tensor v, Tensor out, Tensor dout, Tensor lse, Tensor(a!) delta, Tensor(b!) "
      "dq_accum, Tensor(c!) dk, Tensor(d!) dv, int B, int T, int H, int Hkv, int D, int Dv, float scale, bool causal) "
      "-> ()",
      &attn_bwd_wide);
  m.def(
      "attn_decode(Tensor q, Tensor kcache, Tensor vcache, Tensor? pos, int len, int len_add, int H, float scale, "
      "Tensor(a!) part_o, Tensor(b!) part_ml, Tensor(c!) out) -> ()",
      &attn_decode);
  m.def(
      "attn_decode_paged(Tensor q, Tensor pool, Tensor block_table, Tensor seq_ids, Tensor seq_lens, int len_add, int H, "
      "int Hkv, float scale, Tensor(a!) part_o, Tensor(b!) part_ml, Tensor(c!) out) -> ()",
      &attn_decode_paged);
  m.def("attn_bwd_probs(Tensor(a!) s, Tensor(b!) dp, Tensor lse, Tensor delta, int c, int q0, float scale, bool causal) -> ()", &attn_bwd_probs);
  m.def("norm_bwd_scratch_floats(int D) -> int", [](int64_t D) { return b200::norm_bwd_scratch_floats(static_cast<int>(D)); });
  m.def("gemm_uses_pair(int M, int N, int split_k) -> bool", [](int64_t M, int64_t N, int64_t split_k) {
    b200::GemmArgs a{};
    a.M = static_cast<int>(M);
    a.N = static_cast<int>(N);
    a.split_k = static_cast<int>(split_k);
    return b200::gemm_pair_wanted(a);
  });
  b200_register_extra(m);
  b200_register_runtime(m);
}
