// The Qwen-shaped LoRA training step behind the C ABI: forward, loss, backward, gradient exchange and AdamW as
// calls a host in any language can make (mcb_qwen_*), with no Python, no autograd and no allocation inside a step.
//
// Host code only: it sequences the library's own entry points (the fused LoRA linears, RMSNorm, fused attention,
// SwiGLU, chunked cross-entropy, AdamW, the communicator) exactly as TrainingStep::execute
// (src/training/trainer.rs:368-414) sequences forward_fn, cross_entropy_loss, backward and the optimizer over
// Qwen::forward (src/models/qwen.rs:95-143,236-251), with the backward pass written out because there is no
// autograd.  Everything is enqueued on the caller's stream and can be recorded into a CUDA graph.
//
// Memory: the caller hands over one device arena.  Its head holds what is derived from the weights once (the
// [in,out] copies the backward GEMMs read, the stacked q/k/v weight, the interleaved gate/up weight, AdamW
// moments); the rest is cut afresh for every step: the activations the backward needs, layer by layer, and a
// scratch stack for everything shorter-lived.  The production configuration only: bfloat16, head_dim 64, sequence
// a multiple of 128 (what the fused attention kernels take), MLP width a multiple of 128.
#include <string.h>

#include <vector>

#include "lora_internal.cuh"

using namespace mcb;

namespace {

enum Module { kQ = 0, kK, kV, kO, kGate, kUp, kDown, kModules };

inline size_t up1k(size_t v) { return (v + 1023) & ~static_cast<size_t>(1023); }

// A bump allocator over [base, base + size): null base = a dry run that only measures.
struct Bump {
  uint8_t* base = nullptr;
  size_t size = 0, off = 0, peak = 0;
  bool overflow = false;
  void* take(size_t bytes) {
    const size_t at = off;
    off += up1k(bytes);
    if (off > peak) peak = off;
    if (base != nullptr && off > size) { overflow = true; return nullptr; }
    return base ? base + at : nullptr;
  }
  template <typename T>
  T* take_n(size_t n) { return static_cast<T*>(take(n * sizeof(T))); }
};

struct Adapter {
  const float* A = nullptr;
  const float* B = nullptr;
  float* dA = nullptr;
  float* dB = nullptr;
  float *mA = nullptr, *vA = nullptr, *mB = nullptr, *vB = nullptr;   // AdamW moments (arena)
};

struct LayerState {
  const __nv_bfloat16 *ln1, *ln2;
  const __nv_bfloat16* w[kModules];
  const __nv_bfloat16* wt[kModules];      // [in,out] copies (o, gate, up, down; q/k/v use wqkv_t)
  const __nv_bfloat16 *wqkv, *wqkv_t, *bqkv;
  const __nv_bfloat16* wgu;               // gate/up interleaved in blocks of 128 rows, or null
  Adapter ad[kModules];
};

struct Saved {   // what one layer's backward needs from its forward
  __nv_bfloat16 *h, *n1, *Qr, *Kr, *Vr, *o, *h2, *n2, *gate, *up, *act;
  float* lse;
  __nv_bfloat16 *hqkv, *ho, *hg, *hu, *hd;
};

}  // namespace

struct mcb_qwen {
  mcb_qwen_config cfg;
  int64_t max_tokens = 0;
  int rank = 0;
  float scale = 1.0f;
  int64_t H = 0, I = 0, KV = 0, V = 0, d = 0, W3 = 0;
  int G = 0;
  const __nv_bfloat16 *embed = nullptr, *final_norm = nullptr, *lm_head = nullptr, *lm_head_t = nullptr;
  std::vector<LayerState> layers;
  std::vector<mcb_qwen_adapter_entry> order;   // adapters in the caller's order (AdamW visits them so)
  uint8_t* arena = nullptr;
  size_t arena_bytes = 0, persistent_bytes = 0;
  int64_t ce_chunk = 0;   // tokens per lm_head + loss chunk; 0: mcb_ce_chunk_tokens picks it
  int64_t adamw_steps = 0;                      // the shared counter: one tick per tensor update
  // gradient exchange (optional)
  mcb_comm* comm = nullptr;
  cudaStream_t side = nullptr;
  cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
  float* grad_flat = nullptr;
  std::vector<int64_t> bucket_lo, bucket_hi;
  std::vector<int> bucket_layer;
  int32_t* count = nullptr;   // device: targets kept in the last forward_backward
};

namespace {

size_t ws_bytes_for(const mcb_qwen* q, int64_t M) {
  size_t w = 0;
  auto mx = [&](size_t v) { if (v > w) w = v; };
  const int r = q->rank;
  if (r > 0) {
    mx(mcb_lora_fused_workspace_bytes(M, q->H, q->W3, r, 3, MCB_BF16));
    mx(mcb_lora_workspace_bytes(M, q->H, q->H, r, MCB_BF16));
    mx(mcb_lora_workspace_bytes(M, q->H, q->I, r, MCB_BF16));
    mx(mcb_lora_workspace_bytes(M, q->I, q->H, r, MCB_BF16));
  }
  return w + 1024;
}

bool has(const LayerState& L, int m) { return L.ad[m].A != nullptr; }

// ---- the persistent head of the arena --------------------------------------------------------------------------
int build_persistent(mcb_qwen* q, const mcb_qwen_weights* w, Bump& b, cudaStream_t st) {
  const int64_t H = q->H, I = q->I, KV = q->KV, V = q->V;
  const int64_t out_f[kModules] = {H, KV, KV, H, I, I, H};
  const int64_t in_f[kModules] = {H, H, H, H, H, H, I};
  const bool real = b.base != nullptr;
  auto transpose = [&](const void* src, int64_t rows, int64_t cols) -> const __nv_bfloat16* {
    __nv_bfloat16* dst = b.take_n<__nv_bfloat16>(static_cast<size_t>(rows) * cols);
    if (real && dst) { if (mcb_transpose_2d(src, dst, rows, cols, MCB_BF16, st) != MCB_OK) return nullptr; }
    return dst;
  };
  q->lm_head_t = transpose(w ? w->lm_head : nullptr, V, H);
  for (size_t li = 0; li < q->layers.size(); ++li) {
    LayerState& L = q->layers[li];
    // stacked q/k/v weight and bias
    __nv_bfloat16* cat = b.take_n<__nv_bfloat16>(static_cast<size_t>(q->W3) * H);
    __nv_bfloat16* bc = b.take_n<__nv_bfloat16>(static_cast<size_t>(q->W3));
    if (real && cat && bc) {
      int64_t row = 0;
      for (int m = kQ; m <= kV; ++m) {
        MCB_CHECK_CUDA(cudaMemcpyAsync(cat + row * H, L.w[m], static_cast<size_t>(out_f[m]) * H * 2, cudaMemcpyDeviceToDevice, st));
        const void* bias = w->layers[li].bias[m];
        if (bias) MCB_CHECK_CUDA(cudaMemcpyAsync(bc + row, bias, static_cast<size_t>(out_f[m]) * 2, cudaMemcpyDeviceToDevice, st));
        else MCB_CHECK_CUDA(cudaMemsetAsync(bc + row, 0, static_cast<size_t>(out_f[m]) * 2, st));
        row += out_f[m];
      }
    }
    L.wqkv = cat; L.bqkv = bc;
    L.wqkv_t = transpose(cat, q->W3, H);
    for (int m = kO; m <= kDown; ++m) L.wt[m] = transpose(L.w[m], out_f[m], in_f[m]);
    L.wgu = nullptr;
    if (!has(L, kGate) && !has(L, kUp) && I % 128 == 0) {
      __nv_bfloat16* gu = b.take_n<__nv_bfloat16>(static_cast<size_t>(2 * I) * H);
      if (real && gu) {
        const size_t blk = static_cast<size_t>(128) * H * 2;
        for (int64_t bl = 0; bl < I / 128; ++bl) {
          MCB_CHECK_CUDA(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(gu) + (2 * bl) * blk,
                                         reinterpret_cast<const uint8_t*>(L.w[kGate]) + bl * blk, blk, cudaMemcpyDeviceToDevice, st));
          MCB_CHECK_CUDA(cudaMemcpyAsync(reinterpret_cast<uint8_t*>(gu) + (2 * bl + 1) * blk,
                                         reinterpret_cast<const uint8_t*>(L.w[kUp]) + bl * blk, blk, cudaMemcpyDeviceToDevice, st));
        }
      }
      L.wgu = gu;
    }
    // AdamW moments of this layer's adapters
    for (int m = 0; m < kModules; ++m) {
      if (!has(L, m)) continue;
      const size_t nA = static_cast<size_t>(in_f[m]) * q->rank, nB = static_cast<size_t>(q->rank) * out_f[m];
      Adapter& a = L.ad[m];
      a.mA = b.take_n<float>(nA); a.vA = b.take_n<float>(nA);
      a.mB = b.take_n<float>(nB); a.vB = b.take_n<float>(nB);
      if (real && a.vB) {
        MCB_CHECK_CUDA(cudaMemsetAsync(a.mA, 0, nA * 4, st)); MCB_CHECK_CUDA(cudaMemsetAsync(a.vA, 0, nA * 4, st));
        MCB_CHECK_CUDA(cudaMemsetAsync(a.mB, 0, nB * 4, st)); MCB_CHECK_CUDA(cudaMemsetAsync(a.vB, 0, nB * 4, st));
      }
    }
  }
  q->count = b.take_n<int32_t>(256);
  return MCB_OK;
}

// ---- one step's worth of arena, cut in the order the step uses it ------------------------------------------------
struct StepPlan {
  std::vector<Saved> saved;
  __nv_bfloat16 *h_final = nullptr, *nf = nullptr, *dnf = nullptr;
  float* nll = nullptr;
  float* lossbuf = nullptr;
  void* ws = nullptr; size_t ws_bytes = 0;
  void* attn_ws = nullptr; size_t attn_ws_bytes = 0;
  // scratch shared by all layers (each holds one layer's transient tensors; sized for the largest use)
  __nv_bfloat16 *qkv = nullptr, *t_MH[4] = {nullptr, nullptr, nullptr, nullptr}, *t_MI[2] = {nullptr, nullptr};
  __nv_bfloat16 *dQ = nullptr, *dK = nullptr, *dV = nullptr, *logits = nullptr;
};

void plan_step(const mcb_qwen* q, Bump& b, int64_t M, int64_t B, int64_t S, StepPlan* p) {
  const int64_t H = q->H, I = q->I, KV = q->KV;
  const int r = q->rank;
  const size_t hrow = static_cast<size_t>(mcb_lora_h_pitch(M));
  p->saved.resize(q->layers.size());
  for (size_t li = 0; li < q->layers.size(); ++li) {
    const LayerState& L = q->layers[li];
    Saved& s = p->saved[li];
    memset(&s, 0, sizeof(s));
    s.h = b.take_n<__nv_bfloat16>(M * H);
    s.n1 = b.take_n<__nv_bfloat16>(M * H);
    s.Qr = b.take_n<__nv_bfloat16>(M * H);
    s.Kr = b.take_n<__nv_bfloat16>(M * KV);
    s.Vr = b.take_n<__nv_bfloat16>(M * KV);
    s.lse = b.take_n<float>(static_cast<size_t>(B) * q->cfg.num_heads * S);
    s.o = b.take_n<__nv_bfloat16>(M * H);
    s.h2 = b.take_n<__nv_bfloat16>(M * H);
    if (has(L, kGate) || has(L, kUp)) s.n2 = b.take_n<__nv_bfloat16>(M * H);
    s.gate = b.take_n<__nv_bfloat16>(M * I);
    s.up = b.take_n<__nv_bfloat16>(M * I);
    if (has(L, kDown)) s.act = b.take_n<__nv_bfloat16>(M * I);
    const int nq = (has(L, kQ) ? 1 : 0) + (has(L, kK) ? 1 : 0) + (has(L, kV) ? 1 : 0);
    if (nq > 0) s.hqkv = b.take_n<__nv_bfloat16>(static_cast<size_t>(mcb_lora_rank_padded(static_cast<int64_t>(r) * nq)) * hrow);
    const size_t h1 = static_cast<size_t>(mcb_lora_rank_padded(r)) * hrow;
    if (has(L, kO)) s.ho = b.take_n<__nv_bfloat16>(h1);
    if (has(L, kGate)) s.hg = b.take_n<__nv_bfloat16>(h1);
    if (has(L, kUp)) s.hu = b.take_n<__nv_bfloat16>(h1);
    if (has(L, kDown)) s.hd = b.take_n<__nv_bfloat16>(h1);
  }
  p->h_final = b.take_n<__nv_bfloat16>(M * H);
  p->nf = b.take_n<__nv_bfloat16>(M * H);
  p->dnf = b.take_n<__nv_bfloat16>(M * H);
  p->nll = b.take_n<float>(M);
  p->lossbuf = b.take_n<float>(256);
  p->ws_bytes = ws_bytes_for(q, M);
  p->ws = b.take(p->ws_bytes);
  p->attn_ws_bytes = mcb_attention_workspace_bytes(B * q->cfg.num_kv_heads, q->G, S, q->d);
  p->attn_ws = b.take(p->attn_ws_bytes);
  p->qkv = b.take_n<__nv_bfloat16>(M * q->W3);
  for (int i = 0; i < 4; ++i) p->t_MH[i] = b.take_n<__nv_bfloat16>(M * H);
  for (int i = 0; i < 2; ++i) p->t_MI[i] = b.take_n<__nv_bfloat16>(M * I);
  p->dQ = b.take_n<__nv_bfloat16>(M * H);
  p->dK = b.take_n<__nv_bfloat16>(M * KV);
  p->dV = b.take_n<__nv_bfloat16>(M * KV);
  const int64_t want = q->ce_chunk > 0 ? q->ce_chunk : mcb_ce_chunk_tokens(M, H);
  const int64_t chunk = want < M ? want : M;
  p->logits = b.take_n<__nv_bfloat16>(static_cast<size_t>(chunk) * q->V);
}

#define QCHECK(expr)            \
  do {                          \
    const int rc_ = (expr);     \
    if (rc_ != MCB_OK) return rc_; \
  } while (0)

// y = x W^T (+bias) (+residual) + LoRA, one projection
int lin_fwd(const mcb_qwen* q, const StepPlan& p, const void* x, const void* W, const void* bias, const Adapter& a, const void* residual,
            void* y, void* h_save, int64_t M, int64_t K, int64_t N, cudaStream_t st) {
  const int r = a.A ? q->rank : 0;
  return mcb_lora_linear_fwd_ex(x, W, bias, a.A, a.B, residual, y, r ? h_save : nullptr, M, K, N, r, q->scale, MCB_BF16, MCB_W_OUT_IN,
                                p.ws, p.ws_bytes, st);
}
int lin_bwd(const mcb_qwen* q, const StepPlan& p, const void* x, const void* Wt, const Adapter& a, const void* dy, const void* h_save,
            const void* dx_residual, void* dx, int accumulate, int64_t M, int64_t K, int64_t N, cudaStream_t st) {
  const int r = a.A ? q->rank : 0;
  return mcb_lora_linear_bwd_ex(r ? x : nullptr, Wt, a.A, a.B, dy, r ? h_save : nullptr, dx_residual, dx, r ? a.dA : nullptr,
                                r ? a.dB : nullptr, accumulate, M, K, N, r, q->scale, MCB_BF16, MCB_W_IN_OUT, p.ws, p.ws_bytes, st);
}

int qkv_segments(const mcb_qwen* q, const LayerState& L, mcb_lora_segment* segs) {
  const int64_t off[3] = {0, q->H, q->H + q->KV};
  const int64_t wid[3] = {q->H, q->KV, q->KV};
  int n = 0;
  for (int m = kQ; m <= kV; ++m) {
    if (!has(L, m)) continue;
    segs[n].A = L.ad[m].A; segs[n].B = L.ad[m].B; segs[n].dA = L.ad[m].dA; segs[n].dB = L.ad[m].dB;
    segs[n].n_offset = off[m]; segs[n].n = wid[m];
    ++n;
  }
  return n;
}

int layer_forward(const mcb_qwen* q, const StepPlan& p, size_t li, const __nv_bfloat16* h_in, __nv_bfloat16* h_out, int64_t B, int64_t S,
                  cudaStream_t st) {
  const LayerState& L = q->layers[li];
  const Saved& s = p.saved[li];
  const int64_t M = B * S, H = q->H, I = q->I, KV = q->KV, W3 = q->W3;
  const float eps = q->cfg.rms_norm_eps, theta = q->cfg.rope_theta;
  const int Hq = static_cast<int>(q->cfg.num_heads), Hk = static_cast<int>(q->cfg.num_kv_heads);
  QCHECK(mcb_rmsnorm_fwd(h_in, L.ln1, s.n1, nullptr, M, H, eps, MCB_BF16, st));
  mcb_lora_segment segs[3];
  const int nseg = qkv_segments(q, L, segs);
  if (nseg > 0)
    QCHECK(mcb_lora_linear_fused_fwd(s.n1, L.wqkv, L.bqkv, segs, nseg, p.qkv, s.hqkv, M, H, W3, q->rank, q->scale, MCB_BF16, p.ws,
                                     p.ws_bytes, st));
  else
    QCHECK(mcb_lora_linear_fwd_ex(s.n1, L.wqkv, L.bqkv, nullptr, nullptr, nullptr, p.qkv, nullptr, M, H, W3, 0, 1.0f, MCB_BF16,
                                  MCB_W_OUT_IN, p.ws, p.ws_bytes, st));
  QCHECK(mcb_rope_relayout_qkv(p.qkv, s.Qr, s.Kr, s.Vr, B, S, Hq, Hk, q->d, theta, 0, W3, MCB_BF16, st));
  const float sc = 1.0f / sqrtf(static_cast<float>(q->d));
  QCHECK(mcb_attention_causal_fwd_ex(s.Qr, s.Kr, s.Vr, s.o, s.lse, B * Hk, q->G, S, q->d, sc, MCB_BF16, Hk, 1, p.attn_ws, p.attn_ws_bytes,
                                     st));
  QCHECK(lin_fwd(q, p, s.o, L.w[kO], nullptr, L.ad[kO], h_in, s.h2, s.ho, M, H, H, st));
  __nv_bfloat16* n2 = s.n2 ? s.n2 : p.t_MH[0];
  QCHECK(mcb_rmsnorm_fwd(s.h2, L.ln2, n2, nullptr, M, H, eps, MCB_BF16, st));
  __nv_bfloat16* act = s.act ? s.act : p.t_MI[0];
  if (L.wgu != nullptr) {
    QCHECK(mcb_linear_swiglu_fwd(n2, L.wgu, s.gate, s.up, act, M, H, I, MCB_BF16, st));
  } else {
    QCHECK(lin_fwd(q, p, n2, L.w[kGate], nullptr, L.ad[kGate], nullptr, s.gate, s.hg, M, H, I, st));
    QCHECK(lin_fwd(q, p, n2, L.w[kUp], nullptr, L.ad[kUp], nullptr, s.up, s.hu, M, H, I, st));
    QCHECK(mcb_swiglu_fwd(s.gate, s.up, act, M * I, MCB_BF16, st));
  }
  QCHECK(lin_fwd(q, p, act, L.w[kDown], nullptr, L.ad[kDown], s.h2, h_out, s.hd, M, I, H, st));
  return MCB_OK;
}

// dh_in: gradient of the layer's output [M,H]; dh_out: gradient of its input
int layer_backward(const mcb_qwen* q, const StepPlan& p, size_t li, const __nv_bfloat16* dh3, __nv_bfloat16* dh_out, int64_t B, int64_t S,
                   int accumulate, cudaStream_t st) {
  const LayerState& L = q->layers[li];
  const Saved& s = p.saved[li];
  const int64_t M = B * S, H = q->H, I = q->I, KV = q->KV, W3 = q->W3;
  const float eps = q->cfg.rms_norm_eps, theta = q->cfg.rope_theta;
  const int Hq = static_cast<int>(q->cfg.num_heads), Hk = static_cast<int>(q->cfg.num_kv_heads);
  // MLP
  {
    const Adapter& ad = L.ad[kDown];
    const int r = ad.A ? q->rank : 0;
    if (mcb_lora_linear_bwd_swiglu_supported(M, I, H, r, MCB_BF16)) {
      // the SwiGLU backward runs in the epilogue of the input-gradient GEMM: gate <- d gate, up <- d up, no d act
      QCHECK(mcb_lora_linear_bwd_swiglu(r ? s.act : nullptr, L.wt[kDown], ad.A, ad.B, dh3, r ? s.hd : nullptr, s.gate, s.up,
                                        r ? ad.dA : nullptr, r ? ad.dB : nullptr, accumulate, M, I, H, r, q->scale, MCB_BF16,
                                        MCB_W_IN_OUT, p.ws, p.ws_bytes, st));
    } else {
      __nv_bfloat16* dact = p.t_MI[1];
      QCHECK(lin_bwd(q, p, s.act, L.wt[kDown], ad, dh3, s.hd, nullptr, dact, accumulate, M, I, H, st));
      QCHECK(mcb_swiglu_bwd(s.gate, s.up, dact, s.gate, s.up, M * I, MCB_BF16, st));   // in place: gate <- d gate, up <- d up
    }
  }
  __nv_bfloat16 *dn2a = p.t_MH[1], *dn2 = p.t_MH[2];
  QCHECK(lin_bwd(q, p, s.n2, L.wt[kGate], L.ad[kGate], s.gate, s.hg, nullptr, dn2a, accumulate, M, H, I, st));
  QCHECK(lin_bwd(q, p, s.n2, L.wt[kUp], L.ad[kUp], s.up, s.hu, dn2a, dn2, accumulate, M, H, I, st));
  __nv_bfloat16* dh2 = p.t_MH[3];
  QCHECK(mcb_rmsnorm_bwd_ex(s.h2, L.ln2, dn2, dh3, dh2, nullptr, 0, M, H, eps, MCB_BF16, nullptr, 0, st));
  // attention
  __nv_bfloat16* d_o = p.t_MH[1];
  QCHECK(lin_bwd(q, p, s.o, L.wt[kO], L.ad[kO], dh2, s.ho, nullptr, d_o, accumulate, M, H, H, st));
  const float sc = 1.0f / sqrtf(static_cast<float>(q->d));
  QCHECK(mcb_attention_causal_bwd_ex(s.Qr, s.Kr, s.Vr, s.o, d_o, s.lse, p.dQ, p.dK, p.dV, B * Hk, q->G, S, q->d, sc, MCB_BF16, Hk, 1,
                                     p.attn_ws, p.attn_ws_bytes, st));
  __nv_bfloat16* dqkv = p.qkv;
  QCHECK(mcb_rope_relayout_qkv(dqkv, p.dQ, p.dK, p.dV, B, S, Hq, Hk, q->d, theta, 1, W3, MCB_BF16, st));
  __nv_bfloat16* dn1 = p.t_MH[2];
  mcb_lora_segment segs[3];
  const int nseg = qkv_segments(q, L, segs);
  if (nseg > 0)
    QCHECK(mcb_lora_linear_fused_bwd(s.n1, L.wqkv_t, segs, nseg, dqkv, s.hqkv, nullptr, dn1, accumulate, M, H, W3, q->rank, q->scale,
                                     MCB_BF16, p.ws, p.ws_bytes, st));
  else
    QCHECK(mcb_lora_linear_bwd_ex(nullptr, L.wqkv_t, nullptr, nullptr, dqkv, nullptr, nullptr, dn1, nullptr, nullptr, 0, M, H, W3, 0, 1.0f,
                                  MCB_BF16, MCB_W_IN_OUT, p.ws, p.ws_bytes, st));
  QCHECK(mcb_rmsnorm_bwd_ex(s.h, L.ln1, dn1, dh2, dh_out, nullptr, 0, M, H, eps, MCB_BF16, nullptr, 0, st));
  return MCB_OK;
}

}  // namespace

// ---- C ABI -------------------------------------------------------------------------------------------------------

namespace {
int fill(mcb_qwen* q, const mcb_qwen_config* cfg, const mcb_qwen_weights* w, const mcb_qwen_adapter_entry* adapters, int n_adapters,
         int rank, float scale) {
  q->cfg = *cfg;
  q->H = cfg->hidden_size; q->I = cfg->intermediate_size; q->V = cfg->vocab_size;
  if (cfg->num_heads <= 0 || cfg->num_kv_heads <= 0 || cfg->hidden_size % cfg->num_heads != 0 || cfg->num_heads % cfg->num_kv_heads != 0)
    return fail(MCB_ERR_SHAPE, "mcb_qwen: %lld heads / %lld kv heads do not divide hidden %lld", (long long)cfg->num_heads,
                (long long)cfg->num_kv_heads, (long long)cfg->hidden_size);
  q->d = cfg->hidden_size / cfg->num_heads;
  q->KV = cfg->num_kv_heads * q->d;
  q->G = static_cast<int>(cfg->num_heads / cfg->num_kv_heads);
  q->W3 = q->H + 2 * q->KV;
  if (q->d != 64) return fail(MCB_ERR_UNSUPPORTED, "mcb_qwen: head_dim %lld (the fused attention kernels take 64)", (long long)q->d);
  if (q->H % 8 != 0 || q->I % 8 != 0 || q->V % 8 != 0) return fail(MCB_ERR_ALIGN, "mcb_qwen: widths must be multiples of 8");
  if (rank < 0 || rank > 21 * 3) return fail(MCB_ERR_SHAPE, "mcb_qwen: rank %d", rank);
  if (rank * 3 > 64) return fail(MCB_ERR_UNSUPPORTED, "mcb_qwen: rank %d x 3 fused projections exceeds 64 rank columns", rank);
  q->rank = rank; q->scale = scale;
  q->layers.resize(static_cast<size_t>(cfg->num_layers));
  for (size_t li = 0; li < q->layers.size(); ++li) {
    LayerState& L = q->layers[li];
    L = LayerState();
    if (w) {
      L.ln1 = static_cast<const __nv_bfloat16*>(w->layers[li].input_layernorm);
      L.ln2 = static_cast<const __nv_bfloat16*>(w->layers[li].post_attention_layernorm);
      for (int m = 0; m < kModules; ++m) L.w[m] = static_cast<const __nv_bfloat16*>(w->layers[li].weight[m]);
    }
  }
  q->order.assign(adapters, adapters + n_adapters);
  for (int i = 0; i < n_adapters; ++i) {
    const mcb_qwen_adapter_entry& e = adapters[i];
    if (e.layer < 0 || e.layer >= cfg->num_layers || e.module < 0 || e.module >= kModules)
      return fail(MCB_ERR_SHAPE, "mcb_qwen: adapter %d names layer %d module %d", i, e.layer, e.module);
    if (rank == 0) return fail(MCB_ERR_SHAPE, "mcb_qwen: adapters given but rank is 0");
    Adapter& a = q->layers[e.layer].ad[e.module];
    if (a.A != nullptr) return fail(MCB_ERR_SHAPE, "mcb_qwen: two adapters for layer %d module %d", e.layer, e.module);
    if (w && (!e.A || !e.B || !e.dA || !e.dB)) return fail(MCB_ERR_NULL, "mcb_qwen: adapter %d has a null tensor", i);
    a.A = e.A ? e.A : reinterpret_cast<const float*>(1); a.B = e.B; a.dA = e.dA; a.dB = e.dB;
  }
  return MCB_OK;
}
}  // namespace

extern "C" size_t mcb_qwen_arena_bytes(const mcb_qwen_config* cfg, const mcb_qwen_adapter_entry* adapters, int n_adapters, int rank,
                                       int64_t batch, int64_t seq) {
  if (!cfg || batch <= 0 || seq <= 0 || (n_adapters > 0 && !adapters)) return 0;
  mcb_qwen q;
  if (fill(&q, cfg, nullptr, adapters, n_adapters, rank, 1.0f) != MCB_OK) return 0;
  Bump b;
  if (build_persistent(&q, nullptr, b, nullptr) != MCB_OK) return 0;
  StepPlan p;
  plan_step(&q, b, batch * seq, batch, seq, &p);
  return b.peak + 4096;
}

extern "C" int mcb_qwen_create(mcb_qwen** out, const mcb_qwen_config* cfg, const mcb_qwen_weights* weights,
                               const mcb_qwen_adapter_entry* adapters, int n_adapters, int rank, float scale, void* arena,
                               size_t arena_bytes, void* stream) {
  if (!out || !cfg || !weights || !weights->layers || !arena) return fail(MCB_ERR_NULL, "mcb_qwen_create: null pointer");
  *out = nullptr;
  if ((reinterpret_cast<uintptr_t>(arena) & 1023u) != 0) return fail(MCB_ERR_ALIGN, "mcb_qwen_create: the arena must be 1024-byte aligned");
  if (!current_device_state()) return MCB_ERR_NOT_INIT;
  mcb_qwen* q = new mcb_qwen();
  int rc = fill(q, cfg, weights, adapters, n_adapters, rank, scale);
  if (rc != MCB_OK) { delete q; return rc; }
  q->embed = static_cast<const __nv_bfloat16*>(weights->embed_tokens);
  q->final_norm = static_cast<const __nv_bfloat16*>(weights->final_norm);
  q->lm_head = static_cast<const __nv_bfloat16*>(weights->lm_head);
  if (!q->embed || !q->final_norm || !q->lm_head) { delete q; return fail(MCB_ERR_NULL, "mcb_qwen_create: embed / norm / lm_head is null"); }
  q->arena = static_cast<uint8_t*>(arena); q->arena_bytes = arena_bytes;
  Bump b;
  b.base = q->arena; b.size = arena_bytes;
  rc = build_persistent(q, weights, b, static_cast<cudaStream_t>(stream));
  if (rc == MCB_OK && b.overflow) rc = fail(MCB_ERR_WORKSPACE, "mcb_qwen_create: the arena (%zu bytes) cannot hold the derived weights", arena_bytes);
  if (rc != MCB_OK) { delete q; return rc; }
  q->persistent_bytes = b.off;
  if (cudaEventCreateWithFlags(&q->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
      cudaEventCreateWithFlags(&q->ev_join, cudaEventDisableTiming) != cudaSuccess) {
    delete q;
    return fail(MCB_ERR_UNSUPPORTED, "mcb_qwen_create: cannot create events");
  }
  *out = q;
  return MCB_OK;
}

extern "C" int mcb_qwen_set_exchange(mcb_qwen* q, mcb_comm* comm, void* side_stream, float* grad_flat, const int64_t* bucket_lo,
                                     const int64_t* bucket_hi, const int* bucket_first_layer, int n_buckets) {
  if (!q) return fail(MCB_ERR_NULL, "mcb_qwen_set_exchange: null engine");
  q->comm = comm; q->side = static_cast<cudaStream_t>(side_stream); q->grad_flat = grad_flat;
  q->bucket_lo.clear(); q->bucket_hi.clear(); q->bucket_layer.clear();
  if (comm == nullptr) return MCB_OK;
  if (!grad_flat || !bucket_lo || !bucket_hi || !bucket_first_layer || n_buckets <= 0 || !side_stream)
    return fail(MCB_ERR_NULL, "mcb_qwen_set_exchange: buckets, gradient buffer and side stream are required with a communicator");
  q->bucket_lo.assign(bucket_lo, bucket_lo + n_buckets);
  q->bucket_hi.assign(bucket_hi, bucket_hi + n_buckets);
  q->bucket_layer.assign(bucket_first_layer, bucket_first_layer + n_buckets);
  return MCB_OK;
}

// The lm_head backward is a GEMM of `tokens` rows by `hidden` columns over a very long reduction (the vocabulary):
// few tiles (256 tokens x up to 256 columns each), every one as long as the whole vocabulary, so what decides its
// time is how many WAVES of tiles the CTA pairs need.  Among the chunk sizes of 4096..12288 tokens (multiples of
// 256) this returns the one with the fewest waves over all `tokens` (the smallest of those): 9472 for 32768 tokens
// of width 896 on 148 SMs (37 x 4 = 148 tiles = two full waves; 8192 gives 128 tiles, a wave and three quarters).
extern "C" int64_t mcb_ce_chunk_tokens(int64_t tokens, int64_t hidden) {
  if (tokens <= 0 || hidden <= 0) return 0;
  const DeviceState* ds = current_device_state();
  const int64_t pairs = (ds ? ds->sm_count : 148) / 2;
  const int64_t nt = (hidden + 255) / 256;
  auto waves = [&](int64_t rows) { return rows <= 0 ? 0 : (((rows + 255) / 256) * nt + pairs - 1) / pairs; };
  if (tokens <= 4096) return tokens;
  int64_t best = 8192, best_waves = -1;
  for (int64_t c = 4096; c <= 12288; c += 256) {
    const int64_t w = (tokens / c) * waves(c) + waves(tokens % c);
    if (best_waves < 0 || w < best_waves) { best = c; best_waves = w; }
  }
  return best;
}

extern "C" int mcb_qwen_set_ce_chunk(mcb_qwen* q, int64_t tokens) {
  if (!q) return fail(MCB_ERR_NULL, "mcb_qwen_set_ce_chunk: null engine");
  if (tokens < 0) return fail(MCB_ERR_SHAPE, "mcb_qwen_set_ce_chunk: %lld tokens", (long long)tokens);
  q->ce_chunk = tokens;
  return MCB_OK;
}

extern "C" int mcb_qwen_forward_backward(mcb_qwen* q, const int32_t* ids, const int32_t* targets, int64_t batch, int64_t seq,
                                         int accumulate, float* loss_out, void* stream) {
  MCB_NVTX_RANGE("mcb_qwen_forward_backward");
  if (!q || !ids || !targets || !loss_out) return fail(MCB_ERR_NULL, "mcb_qwen_forward_backward: null pointer");
  if (batch <= 0 || seq <= 0) return fail(MCB_ERR_SHAPE, "mcb_qwen_forward_backward: batch %lld x seq %lld", (long long)batch, (long long)seq);
  if (seq % 128 != 0) return fail(MCB_ERR_UNSUPPORTED, "mcb_qwen_forward_backward: sequence %lld (the fused attention kernels take multiples of 128)", (long long)seq);
  if (q->order.empty()) return fail(MCB_ERR_SHAPE, "mcb_qwen_forward_backward: no adapters to train");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t M = batch * seq, H = q->H, V = q->V;
  Bump b;
  b.base = q->arena; b.size = q->arena_bytes; b.off = q->persistent_bytes;
  StepPlan p;
  plan_step(q, b, M, batch, seq, &p);
  if (b.overflow) return fail(MCB_ERR_WORKSPACE, "mcb_qwen_forward_backward: the arena (%zu bytes) is too small for %lld x %lld tokens (%zu needed)",
                              q->arena_bytes, (long long)batch, (long long)seq, b.peak);
  const size_t nl = q->layers.size();
  // forward
  QCHECK(mcb_embedding_fwd(ids, q->embed, p.saved[0].h, M, H, V, MCB_BF16, st));
  for (size_t li = 0; li < nl; ++li) {
    __nv_bfloat16* h_out = li + 1 < nl ? p.saved[li + 1].h : p.h_final;
    QCHECK(layer_forward(q, p, li, p.saved[li].h, h_out, batch, seq, st));
  }
  QCHECK(mcb_rmsnorm_fwd(p.h_final, q->final_norm, p.nf, nullptr, M, H, q->cfg.rms_norm_eps, MCB_BF16, st));
  // lm_head, loss and lm_head backward, a chunk of tokens at a time
  QCHECK(mcb_cross_entropy_count(targets, q->count, M, V, st));
  const int64_t want = q->ce_chunk > 0 ? q->ce_chunk : mcb_ce_chunk_tokens(M, H);
  const int64_t chunk = want < M ? want : M;
  for (int64_t c0 = 0; c0 < M; c0 += chunk) {
    const int64_t rows = (M - c0 < chunk) ? M - c0 : chunk;
    QCHECK(mcb_lora_linear_fwd_ex(p.nf + c0 * H, q->lm_head, nullptr, nullptr, nullptr, nullptr, p.logits, nullptr, rows, H, V, 0, 1.0f,
                                  MCB_BF16, MCB_W_OUT_IN, p.ws, p.ws_bytes, st));
    QCHECK(mcb_cross_entropy_chunk(p.logits, targets + c0, p.nll + c0, q->count, rows, V, 1, MCB_BF16, st));
    QCHECK(mcb_lora_linear_bwd_ex(nullptr, q->lm_head_t, nullptr, nullptr, p.logits, nullptr, nullptr, p.dnf + c0 * H, nullptr, nullptr, 0,
                                  rows, H, V, 0, 1.0f, MCB_BF16, MCB_W_IN_OUT, p.ws, p.ws_bytes, st));
  }
  QCHECK(mcb_cross_entropy_finish(p.nll, q->count, loss_out, M, st));
  // backward
  __nv_bfloat16 *dh = p.t_MH[0], *dh_next = p.nf;   // two buffers the layers ping-pong between
  QCHECK(mcb_rmsnorm_bwd_ex(p.h_final, q->final_norm, p.dnf, nullptr, dh, nullptr, 0, M, H, q->cfg.rms_norm_eps, MCB_BF16, nullptr, 0, st));
  bool forked = false;
  for (size_t k = nl; k-- > 0;) {
    QCHECK(layer_backward(q, p, k, dh, dh_next, batch, seq, accumulate, st));
    __nv_bfloat16* t = dh; dh = dh_next; dh_next = t;
    if (q->comm != nullptr) {
      for (size_t bi = 0; bi < q->bucket_layer.size(); ++bi) {
        if (q->bucket_layer[bi] != static_cast<int>(k)) continue;
        // the bucket's gradients are final on this stream: the side stream takes over from here
        MCB_CHECK_CUDA(cudaEventRecord(q->ev_fork, st));
        MCB_CHECK_CUDA(cudaStreamWaitEvent(q->side, q->ev_fork, 0));
        QCHECK(mcb_comm_allreduce_bucket(q->comm, q->grad_flat + q->bucket_lo[bi], q->bucket_hi[bi] - q->bucket_lo[bi], q->side));
        forked = true;
      }
    }
  }
  if (forked) {
    MCB_CHECK_CUDA(cudaEventRecord(q->ev_join, q->side));
    MCB_CHECK_CUDA(cudaStreamWaitEvent(st, q->ev_join, 0));
  }
  return MCB_OK;
}

extern "C" int mcb_qwen_adamw_step(mcb_qwen* q, float lr, float beta1, float beta2, float eps, float weight_decay, float grad_scale,
                                   void* stream) {
  MCB_NVTX_RANGE("mcb_qwen_adamw_step");
  if (!q) return fail(MCB_ERR_NULL, "mcb_qwen_adamw_step: null engine");
  const int64_t in_f[kModules] = {q->H, q->H, q->H, q->H, q->H, q->H, q->I};
  const int64_t out_f[kModules] = {q->H, q->KV, q->KV, q->H, q->I, q->I, q->H};
  std::vector<mcb_adamw_tensor> ts;
  ts.reserve(q->order.size() * 2);
  for (const mcb_qwen_adapter_entry& e : q->order) {
    const Adapter& a = q->layers[e.layer].ad[e.module];
    mcb_adamw_tensor t;
    t.p = const_cast<float*>(a.A); t.g = a.dA; t.m = a.mA; t.v = a.vA; t.n = in_f[e.module] * q->rank;
    t.t = static_cast<int32_t>(++q->adamw_steps); t.pad_ = 0;
    ts.push_back(t);
    t.p = const_cast<float*>(a.B); t.g = a.dB; t.m = a.mB; t.v = a.vB; t.n = static_cast<int64_t>(q->rank) * out_f[e.module];
    t.t = static_cast<int32_t>(++q->adamw_steps);
    ts.push_back(t);
  }
  return mcb_adamw_multi(ts.data(), static_cast<int>(ts.size()), lr, beta1, beta2, eps, weight_decay, grad_scale, stream);
}

extern "C" int mcb_qwen_train_step(mcb_qwen* q, const int32_t* ids, const int32_t* targets, int64_t batch, int64_t seq, float lr,
                                   float beta1, float beta2, float eps, float weight_decay, float grad_scale, float* loss_out,
                                   void* stream) {
  MCB_NVTX_RANGE("mcb_qwen_train_step");
  if (int rc = mcb_qwen_forward_backward(q, ids, targets, batch, seq, 0, loss_out, stream)) return rc;
  return mcb_qwen_adamw_step(q, lr, beta1, beta2, eps, weight_decay, grad_scale, stream);
}

extern "C" int mcb_qwen_info(const mcb_qwen* q, int64_t* adamw_steps, int64_t* persistent_bytes, int32_t** kept_targets_dev) {
  if (!q) return fail(MCB_ERR_NULL, "mcb_qwen_info: null engine");
  if (adamw_steps) *adamw_steps = q->adamw_steps;
  if (persistent_bytes) *persistent_bytes = static_cast<int64_t>(q->persistent_bytes);
  if (kept_targets_dev) *kept_targets_dev = q->count;
  return MCB_OK;
}

extern "C" int mcb_qwen_destroy(mcb_qwen* q) {
  if (!q) return MCB_OK;
  if (q->ev_fork) cudaEventDestroy(q->ev_fork);
  if (q->ev_join) cudaEventDestroy(q->ev_join);
  delete q;
  return MCB_OK;
}
