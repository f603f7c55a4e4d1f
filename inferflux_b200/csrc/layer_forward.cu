// One pre-norm decoder layer (norm, attention with rotation and paged cache, norm, SwiGLU feed-forward)
// launched from native code: the same kernels, chosen by the same rules, as the kernel table in ops.py
// launches one by one when a block's parts call it, but without a trip through the interpreter per kernel.
// A step that is not a CUDA graph (prompt portions, mixed steps) costs about 13 us of host time a launch
// from Python and 2-3 us from here; at the smaller model sizes such steps are bound by exactly that.
//
// The reference's counterpart is the layer loop of LlamaForwardTyped<T>::Forward / BatchForwardDevice
// (runtime/backends/cuda/native/transformer_forward.cu:1792-2600, 3100-3900), which is native too.
//
// Nothing here knows a model: the caller (CudaKernels.fused_prenorm_layer) hands in the sizes and constants of the
// layer's parts.  Temporaries live in a workspace the caller owns; the layer's last delta (the down
// projection, not yet added to the residual stream) is left in one of two regions of it, alternating by
// layer, for whatever normalises next.
#include "common.cuh"

extern "C" {
int ifx_rmsnorm(float*, const void*, const float*, void*, int, int, float, int, int, cudaStream_t);
int ifx_reduce_add_rmsnorm(float*, const float*, const float*, void*, int, int, float, int, float*, int*, int, cudaStream_t);
int ifx_prenorm(float*, const void*, const float*, void*, float*, int, int, int, int, cudaStream_t);
int ifx_silu_mul(const void*, void*, int, int, int, cudaStream_t);
int ifx_gemm_skinny(const void*, const void*, const float*, void*, float*, int, int, int, int, int, int, int, int,
                    const float*, int, float, int*, cudaStream_t);
int ifx_gemm_cublas_bf16(const void*, const void*, void*, int, int, int, int, cudaStream_t);
int ifx_gemm_tcgen05(const void*, const void*, void*, int, int, int, int, int, int, int*, cudaStream_t);
int ifx_rope_append(const void*, const float*, int, const float*, const float*, int, int, const int*, const int*, const int*,
                    const int*, int, int, int, void*, void*, int, int, int, int, int, int, int, cudaStream_t);
int ifx_attention_mma_supports(int);
int ifx_attention_prefill_tcgen05_supports(int, int);
int ifx_attention_prefill_tcgen05(const void*, int, const void*, const int*, const int*, const int*, void*, int, int, int, int,
                                  int, int, int, int, float, int*, cudaStream_t);
int ifx_attention_prefill_bf16(const void*, const void*, const int*, const int*, const int*, void*, int, int, int, int, int,
                               int, int, int, float, int, int*, cudaStream_t);
int ifx_attention_decode_max_splits(int, int);
int ifx_attention_decode_bf16(const void*, const void*, const int*, const int*, void*, int, int, int, int, int, int, int, int,
                              float, int, int, int*, cudaStream_t);
int ifx_attention_generic(const void*, const void*, const int*, const int*, const int*, const int*, const int*, void*, int, int,
                          int, int, int, int, int, int, float, int, cudaStream_t);
}

// The three structures below are mirrored by ctypes structures in ops.py: keep the order of the fields.

// One step's batch: filled once a step, the same for every layer.
struct IfxStepArgs {
  int T, num_decode, num_tiles, max_kv_len;
  const int *positions, *token_req, *req_slot, *decode_rows, *decode_meta, *prefill_tiles;
  float* norm_sumsq;          // [128 * 64] and [128]: scratch of the many-block reduce + norm
  int* norm_tickets;
  int* error_flag;
  // the kernel table's knobs
  int skinny_max_rows, swiglu_tiles, swiglu_tiles_max_k, tensor_core_prefill;
  int overlap_attention, pad0;   // 1: a mixed step's two attention kernels run side by side on two streams
};

// One layer with one cache: filled once, when the layer first runs.
struct IfxLayerArgs {
  int hidden, inter, nq, nkv, d, window, rot, interleaved;
  float scale, eps_in, eps_post;
  int write_cache;
  const float *norm_in_w, *norm_post_w, *b_qkv, *inv_freq;
  const void *w_qkv, *w_o, *w_gate_up, *w_down;
  void* kv_pool;
  const int* block_table;
  int max_blocks, page_size, num_pages, pad0;
};

// What changes from call to call, and what comes back.
struct IfxLayerIO {
  float* x;                   // residual stream, float32 [T, hidden], updated in place
  const void* pending_tensor; // the delta the block before left unadded: bfloat16 [T, hidden],
  const float* pending_parts; //   or float32 K slices [pending_splits, T, hidden], or neither
  int pending_splits, parity; // parity: which of the workspace's two delta regions this call writes
  unsigned char* ws;
  long long ws_bytes;
  void* out_tensor;           // this layer's last delta, unadded: one of the two forms again
  float* out_parts;
  int out_splits, launches, library_calls, pad0;
};

namespace {

constexpr int kChunk = 512;                // columns per chunk of the pre-norm's sums of squares (elementwise.cu)

struct Arena {
  unsigned char* base;
  size_t used, size;
  void* take(size_t bytes) {
    const size_t at = (used + 255) & ~(size_t)255;
    used = at + bytes;
    return used <= size ? base + at : nullptr;
  }
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// The routing rules below restate those of ops.py; tests/test_native_layer_gpu.py holds the two paths to each
// other bit for bit, so a rule changed in one place only shows at once.
// K slices of a few-rows product, as CudaKernels.linear chooses them.
inline int skinny_splits(int T, int N, int K) {
  const int tiles = (N + 127) / 128, kblocks = (K + 63) / 64;
  const int slots = T <= 128 ? 296 : 148, most = T <= 128 ? 10 : 5;
  int s = slots / tiles;
  if (s > most) s = most;
  if (s > kblocks / 4) s = kblocks / 4;
  return s < 1 ? 1 : s;
}

inline int decode_splits(int tokens, int nkv, int max_keys, int max_splits) {
  int want = 296 / (tokens * nkv > 0 ? tokens * nkv : 1);
  if (want < 1) want = 1;
  int limit = want;
  if (limit > max_keys / 128) limit = max_keys / 128;
  if (limit > max_splits) limit = max_splits;
  if (limit < 1) limit = 1;
  int s = 1;
  while (s * 2 <= limit) s *= 2;
  if (s > 8 && tokens * nkv * s > 148) s = 8;
  return s;
}

// Whether the decode attention's grid is small enough to be let in early behind the rotation kernel
// (CudaKernels.small_attention_grid).
inline int small_attention_grid(int num_decode, int num_tiles, int nkv) {
  return num_tiles == 0 && num_decode * nkv * 8 <= 148 ? 1 : 0;
}

// A second stream and two events per device, for the two attention kernels of a mixed step: the one over the
// prompt portions (tensor-bound, few blocks) and the one over the single decoded tokens (HBM-bound) read the same
// queries and write different rows, so neither has to wait for the other.
struct SideStream {
  cudaStream_t stream = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr;
  bool ok = false;
};
inline SideStream* side_stream() {
  static SideStream per_device[16];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 16) return nullptr;
  SideStream& s = per_device[dev];
  if (!s.stream) {
    s.ok = cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) == cudaSuccess &&
           cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) == cudaSuccess;
  }
  return s.ok ? &s : nullptr;
}

struct Delta {               // a product's result on its way to the residual stream
  void* tensor = nullptr;    // bfloat16 [T, N]
  float* parts = nullptr;    // float32 [splits, T, N]
  int splits = 0;
};

struct Call {                // one call's three structures and its workspace
  const IfxStepArgs* s;
  const IfxLayerArgs* l;
  IfxLayerIO* io;
  Arena ws;
  cudaStream_t st;
};

#define RUN(call)            \
  do {                       \
    int rc__ = (call);       \
    if (rc__) return rc__;   \
    ++c.io->launches;        \
  } while (0)

int cublas(Call& c, const void* act, const void* W, void* out, int N, int K) {
  const int rc = ifx_gemm_cublas_bf16(act, W, out, c.s->T, N, K, IFX_DT_BF16, c.st);
  if (!rc) ++c.io->library_calls;
  return rc;
}

// x += delta; h = norm(x).  Few rows: the norm's row scale is left to the product that follows (*scaled), which
// then takes x * w and the per-chunk sums of squares.
int norm_step(Call& c, const Delta& delta, const float* w, float eps, void* h, float* sumsq, bool* scaled) {
  const int T = c.s->T, H = c.l->hidden;
  float* x = c.io->x;
  *scaled = T <= c.s->skinny_max_rows && H % 8 == 0;
  if (*scaled) {
    const void* src = delta.parts ? (const void*)delta.parts : delta.tensor;
    RUN(ifx_prenorm(x, src, w, h, sumsq, T, H, delta.parts ? delta.splits : 0, IFX_DT_BF16, c.st));
    return 0;
  }
  if (delta.parts) {
    const int chunks = (H + kChunk - 1) / kChunk;
    if (T <= 128 && T * chunks <= 128 * 64)
      RUN(ifx_reduce_add_rmsnorm(x, delta.parts, w, h, T, H, eps, delta.splits, c.s->norm_sumsq, c.s->norm_tickets,
                                 IFX_DT_BF16, c.st));
    else
      RUN(ifx_rmsnorm(x, delta.parts, w, h, T, H, eps, delta.splits, IFX_DT_BF16, c.st));
  } else {
    RUN(ifx_rmsnorm(x, delta.tensor, w, h, T, H, eps, 0, IFX_DT_BF16, c.st));
  }
  return 0;
}

// out = act . W^T for a consumer that adds K slices itself (CudaKernels.linear with allow_partial).
// `fixed`: where the result goes (a delta region); else it is taken from the workspace.
int linear_partial(Call& c, const void* act, const void* W, int N, int K, const float* sumsq, float eps, Delta* out,
                   void* fixed) {
  const int T = c.s->T;
  if (T <= c.s->skinny_max_rows && K % 8 == 0 && aligned16(act) && aligned16(W)) {
    const int splits = skinny_splits(T, N, K);
    const int chunks = sumsq ? (K + kChunk - 1) / kChunk : 0;
    if (splits > 1) {
      float* parts = fixed ? (float*)fixed : (float*)c.ws.take((size_t)splits * T * N * 4);
      if (!parts) return IFX_E_TOOBIG;
      RUN(ifx_gemm_skinny(act, W, nullptr, nullptr, parts, T, N, K, N, splits, 1, 0, 0, sumsq, chunks, eps,
                          c.s->error_flag, c.st));
      out->parts = parts;
      out->splits = splits;
      return 0;
    }
    void* t = fixed ? fixed : c.ws.take((size_t)T * N * 2);
    if (!t) return IFX_E_TOOBIG;
    RUN(ifx_gemm_skinny(act, W, nullptr, t, nullptr, T, N, K, N, 1, 0, 0, 0, sumsq, chunks, eps, c.s->error_flag, c.st));
    out->tensor = t;
    return 0;
  }
  if (sumsq) return IFX_E_BADARG;                      // pre-normed rows only ever go to the few-rows product
  void* t = fixed ? fixed : c.ws.take((size_t)T * N * 2);
  if (!t) return IFX_E_TOOBIG;
  const int rc = cublas(c, act, W, t, N, K);
  if (rc) return rc;
  out->tensor = t;
  return 0;
}

inline size_t delta_region_bytes(int T, int hidden, int skinny_max_rows) {
  return T <= skinny_max_rows ? (size_t)10 * T * hidden * 4 : (size_t)T * hidden * 2;     // up to 10 K slices
}

}  // namespace

// Bytes of workspace a layer of these sizes may need for T token rows (both delta regions included).
extern "C" long long ifx_layer_workspace_bytes(int T, int hidden, int q_dim, int kv_dim, int inter, int skinny_max_rows) {
  const bool few = T <= skinny_max_rows;
  auto delta = [&](size_t n) { return (few ? (size_t)10 * T * n * 4 : (size_t)T * n * 2) + 256; };
  const size_t qkv = (size_t)q_dim + 2 * (size_t)kv_dim;
  const size_t chunks = (hidden + kChunk - 1) / kChunk;
  size_t total = 2 * (delta_region_bytes(T, hidden, skinny_max_rows) + 256);
  total += 2 * ((size_t)T * hidden * 2 + 256) + 2 * ((size_t)T * chunks * 4 + 256);      // normed rows, sums of squares
  total += delta(qkv) + 2 * ((size_t)T * q_dim * 2 + 256) + delta(hidden);               // q/k/v, q, attention, o
  total += (size_t)T * 2 * inter * 2 + (size_t)T * inter * 2 + 512;                      // gate|up, activation
  return (long long)total + 1024;
}

extern "C" int ifx_layer_forward(const IfxStepArgs* s, const IfxLayerArgs* l, IfxLayerIO* io, cudaStream_t st) {
  if (!s || !l || !io) return IFX_E_BADARG;
  io->launches = io->library_calls = 0;
  io->out_tensor = nullptr;
  io->out_parts = nullptr;
  io->out_splits = 0;
  if (s->T <= 0) return 0;
  if (!io->x || !io->ws || !l->kv_pool || !l->block_table || !s->error_flag) return IFX_E_BADARG;
  Call c{s, l, io, Arena{io->ws, 0, (size_t)io->ws_bytes}, st};
  const int T = s->T, H = l->hidden, nq = l->nq, nkv = l->nkv, d = l->d, I = l->inter;
  const int q_dim = nq * d, qkv_dim = (nq + 2 * nkv) * d;
  const int chunks = (H + kChunk - 1) / kChunk;

  // the two delta regions come first: this call writes the one of its parity and may read the other
  const size_t region = delta_region_bytes(T, H, s->skinny_max_rows);
  unsigned char* regions[2] = {(unsigned char*)c.ws.take(region), (unsigned char*)c.ws.take(region)};
  if (!regions[0] || !regions[1]) return IFX_E_TOOBIG;
  unsigned char* mine = regions[io->parity & 1];
  Delta pending;
  pending.tensor = const_cast<void*>(io->pending_tensor);
  pending.parts = const_cast<float*>(io->pending_parts);
  pending.splits = io->pending_splits;
  if (pending.tensor == mine || (void*)pending.parts == mine) return IFX_E_BADARG;

  // ---- x += pending; h = norm(x)
  void* h = c.ws.take((size_t)T * H * 2);
  float* sumsq = (float*)c.ws.take((size_t)T * chunks * 4);
  if (!h || !sumsq) return IFX_E_TOOBIG;
  bool scaled = false;
  int rc = norm_step(c, pending, l->norm_in_w, l->eps_in, h, sumsq, &scaled);
  if (rc) return rc;

  // ---- q, k, v = h Wqkv^T; bias, rotation, cache append
  Delta qkv;
  rc = linear_partial(c, h, l->w_qkv, qkv_dim, H, scaled ? sumsq : nullptr, l->eps_in, &qkv, nullptr);
  if (rc) return rc;
  void* q = c.ws.take((size_t)T * q_dim * 2);
  void* attn = c.ws.take((size_t)T * q_dim * 2);
  if (!q || !attn) return IFX_E_TOOBIG;
  RUN(ifx_rope_append(qkv.tensor, qkv.parts, qkv.splits, l->b_qkv, l->inv_freq, l->rot, l->interleaved, s->positions,
                      s->token_req, s->req_slot, l->block_table, l->max_blocks, l->page_size, l->num_pages, l->kv_pool, q, T,
                      nq, nkv, d, l->write_cache ? 1 : 0, small_attention_grid(s->num_decode, s->num_tiles, nkv), IFX_DT_BF16, st));

  // ---- attention over the paged cache: prompt portions in one launch, single decoded tokens in another
  if (ifx_attention_mma_supports(d)) {
    // both kinds in one step: the decoded tokens' kernel goes to the side stream, behind the rotation kernel
    cudaStream_t decode_st = st;
    SideStream* side = nullptr;
    if (s->overlap_attention && s->num_tiles > 0 && s->num_decode > 0 && nq / nkv <= 16) {
      cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
      if (cudaStreamIsCapturing(st, &capturing) == cudaSuccess && capturing == cudaStreamCaptureStatusNone &&
          (side = side_stream()) != nullptr) {
        if (cudaEventRecord(side->fork, st) != cudaSuccess || cudaStreamWaitEvent(side->stream, side->fork, 0) != cudaSuccess)
          return IFX_E_BADARG;
        decode_st = side->stream;
      }
    }
    if (s->num_tiles > 0) {
      if (s->tensor_core_prefill && ifx_attention_prefill_tcgen05_supports(d, l->page_size))
        RUN(ifx_attention_prefill_tcgen05(q, T, l->kv_pool, l->block_table, s->prefill_tiles, s->req_slot, attn, s->num_tiles,
                                          nq, nkv, d, l->page_size, l->max_blocks, l->num_pages, l->window, l->scale,
                                          s->error_flag, st));
      else
        RUN(ifx_attention_prefill_bf16(q, l->kv_pool, l->block_table, s->prefill_tiles, s->req_slot, attn, s->num_tiles, nq,
                                       nkv, d, l->page_size, l->max_blocks, l->num_pages, l->window, l->scale, s->max_kv_len,
                                       s->error_flag, st));
    }
    if (s->num_decode > 0) {
      if (nq / nkv > 16) {
        RUN(ifx_attention_generic(q, l->kv_pool, l->block_table, s->positions, s->token_req, s->req_slot, s->decode_rows,
                                  attn, s->num_decode, nq, nkv, d, l->page_size, l->max_blocks, l->num_pages, l->window,
                                  l->scale, IFX_DT_BF16, st));
      } else {
        const int max_keys = l->window > 0 && l->window < s->max_kv_len ? l->window : s->max_kv_len;
        const int splits = decode_splits(s->num_decode, nkv, max_keys, ifx_attention_decode_max_splits(d, l->page_size));
        RUN(ifx_attention_decode_bf16(q, l->kv_pool, l->block_table, s->decode_meta, attn, s->num_decode, nq, nkv, d,
                                      l->page_size, l->max_blocks, l->num_pages, l->window, l->scale, splits, max_keys,
                                      s->error_flag, decode_st));
      }
    }
    if (decode_st != st &&
        (cudaEventRecord(side->join, decode_st) != cudaSuccess || cudaStreamWaitEvent(st, side->join, 0) != cudaSuccess))
      return IFX_E_BADARG;
  } else {
    RUN(ifx_attention_generic(q, l->kv_pool, l->block_table, s->positions, s->token_req, s->req_slot, nullptr, attn, T, nq,
                              nkv, d, l->page_size, l->max_blocks, l->num_pages, l->window, l->scale, IFX_DT_BF16, st));
  }

  // ---- output projection; x += it; h = norm(x)
  Delta o;
  rc = linear_partial(c, attn, l->w_o, H, q_dim, nullptr, 0.0f, &o, nullptr);
  if (rc) return rc;
  void* h2 = c.ws.take((size_t)T * H * 2);
  float* sumsq2 = (float*)c.ws.take((size_t)T * chunks * 4);
  if (!h2 || !sumsq2) return IFX_E_TOOBIG;
  rc = norm_step(c, o, l->norm_post_w, l->eps_post, h2, sumsq2, &scaled);
  if (rc) return rc;

  // ---- act = silu(h Wg^T) * (h Wu^T)
  void* act = c.ws.take((size_t)T * I * 2);
  if (!act) return IFX_E_TOOBIG;
  if (T <= s->skinny_max_rows && H % 8 == 0 && aligned16(h2) && aligned16(l->w_gate_up)) {
    RUN(ifx_gemm_skinny(h2, l->w_gate_up, nullptr, act, nullptr, T, I, H, 2 * I, 1, 2, I, 0, scaled ? sumsq2 : nullptr,
                        scaled ? chunks : 0, l->eps_post, s->error_flag, st));
  } else if (scaled) {
    return IFX_E_BADARG;
  } else if (s->swiglu_tiles && H % 8 == 0 && H <= s->swiglu_tiles_max_k && aligned16(h2) && aligned16(l->w_gate_up)) {
    RUN(ifx_gemm_tcgen05(h2, l->w_gate_up, act, T, I, H, 2 * I, 1, I, s->error_flag, st));
  } else {
    void* gu = c.ws.take((size_t)T * 2 * I * 2);
    if (!gu) return IFX_E_TOOBIG;
    rc = cublas(c, h2, l->w_gate_up, gu, 2 * I, H);
    if (rc) return rc;
    RUN(ifx_silu_mul(gu, act, T, I, IFX_DT_BF16, st));
  }

  // ---- down projection: left unadded in this call's delta region
  Delta down;
  rc = linear_partial(c, act, l->w_down, H, I, nullptr, 0.0f, &down, mine);
  if (rc) return rc;
  io->out_tensor = down.tensor;
  io->out_parts = down.parts;
  io->out_splits = down.splits;
  return 0;
}
