// Harness around the UNMODIFIED reference sources (anvai-labs/inferflux).
//
// The reference is a C++ server; its dense model path is LlamaForwardTyped<T>
// (runtime/backends/cuda/native/transformer_forward.cu), fed by a weight map, a
// contiguous key/value cache (kv_cache_gpu.cu), cuBLAS (cublas_gemm.cpp) and the
// GPU sampler (gpu_sampler.cu).  This file is NOT reference code: it owns no kernel
// and no model arithmetic.  It makes weights (random, or read from raw files),
// builds the reference's own objects through their public interfaces, and calls
//   ModelForward::Forward       (one prompt portion, transformer_forward.cu:1677)
//   ModelForward::BatchForward  (one token of B sequences, :2911)
//   GpuSampler                  (greedy argmax)
// and the leaf host wrappers of cuda_kernels.cuh / flash_attention.cuh, to
//   * time the reference at a given shape          (mode `bench`),
//   * write the reference's logits of a tiny model (mode `model`),
//   * write the outputs of single wrappers         (mode `leaf`).
// None of the engine's own libraries is linked or loaded here.
//
// Arguments are key=value pairs after the mode.
#include "runtime/backends/cuda/kernels/flash_attention.cuh"
#include "runtime/backends/cuda/native/cublas_gemm.h"
#include "runtime/backends/cuda/native/cuda_kernels.cuh"
#include "runtime/backends/cuda/native/gpu_sampler.h"
#include "runtime/backends/cuda/native/kv_cache_gpu.h"
#include "runtime/backends/cuda/native/model_forward.h"
#include "runtime/backends/cuda/native/model_forward_factory.h"
#include "runtime/backends/cuda/native/native_execution_policy.h"
#include "runtime/backends/cuda/native/weight_map.h"

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

using namespace inferflux;

#define CK(call)                                                                  \
  do {                                                                            \
    cudaError_t e_ = (call);                                                      \
    if (e_ != cudaSuccess) {                                                      \
      std::fprintf(stderr, "ref_harness: %s failed: %s (%s:%d)\n", #call,         \
                   cudaGetErrorString(e_), __FILE__, __LINE__);                   \
      std::exit(3);                                                               \
    }                                                                             \
  } while (0)

static void die(const std::string &msg) {
  std::fprintf(stderr, "ref_harness: %s\n", msg.c_str());
  std::exit(2);
}

// ------------------------------------------------------------------ arguments
struct Args {
  std::map<std::string, std::string> kv;
  bool has(const std::string &k) const { return kv.count(k) > 0; }
  std::string str(const std::string &k, const std::string &def = "") const {
    auto it = kv.find(k);
    return it == kv.end() ? def : it->second;
  }
  long num(const std::string &k, long def) const {
    return has(k) ? std::atol(kv.at(k).c_str()) : def;
  }
  double real(const std::string &k, double def) const {
    return has(k) ? std::atof(kv.at(k).c_str()) : def;
  }
  long need(const std::string &k) const {
    if (!has(k)) die("missing argument " + k + "=");
    return std::atol(kv.at(k).c_str());
  }
};

static Args parse(int argc, char **argv, int first) {
  Args a;
  for (int i = first; i < argc; ++i) {
    std::string s(argv[i]);
    auto eq = s.find('=');
    if (eq == std::string::npos) die("expected key=value, got " + s);
    a.kv[s.substr(0, eq)] = s.substr(eq + 1);
  }
  return a;
}

static std::vector<int> ints(const std::string &csv) {
  std::vector<int> out;
  std::stringstream ss(csv);
  std::string tok;
  while (std::getline(ss, tok, ','))
    if (!tok.empty()) out.push_back(std::atoi(tok.c_str()));
  return out;
}

// ---------------------------------------------------------------------- files
static std::vector<char> read_file(const std::string &path) {
  std::ifstream f(path, std::ios::binary | std::ios::ate);
  if (!f) die("cannot read " + path);
  std::vector<char> buf(static_cast<size_t>(f.tellg()));
  f.seekg(0);
  f.read(buf.data(), static_cast<std::streamsize>(buf.size()));
  return buf;
}

static bool file_exists(const std::string &path) {
  std::ifstream f(path, std::ios::binary);
  return static_cast<bool>(f);
}

static void write_file(const std::string &path, const void *data, size_t bytes) {
  std::ofstream f(path, std::ios::binary);
  if (!f) die("cannot write " + path);
  f.write(static_cast<const char *>(data), static_cast<std::streamsize>(bytes));
}

template <typename T> static T *upload(const std::vector<char> &bytes) {
  T *d = nullptr;
  CK(cudaMalloc(&d, bytes.size() ? bytes.size() : 16));
  CK(cudaMemcpy(d, bytes.data(), bytes.size(), cudaMemcpyHostToDevice));
  return d;
}

template <typename T> static void download_to(const std::string &path, const T *d, size_t count) {
  std::vector<T> h(count);
  CK(cudaMemcpy(h.data(), d, count * sizeof(T), cudaMemcpyDeviceToHost));
  write_file(path, h.data(), count * sizeof(T));
}

static double now_unix() {
  using namespace std::chrono;
  return duration<double>(system_clock::now().time_since_epoch()).count();
}

// -------------------------------------------------------------------- weights
// Made-up weights for timing: N(0, std) from a counter hash, written in T.  The
// values only have to be of the size real weights have; no result is compared.
__device__ __forceinline__ unsigned mix32(unsigned x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}

template <typename T>
__global__ void fill_normal_kernel(T *out, size_t n, unsigned seed, float mean, float std) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  for (; i < n; i += stride) {
    unsigned a = mix32(static_cast<unsigned>(i) * 2u + 1u + seed * 0x9e3779b9U);
    unsigned b = mix32(static_cast<unsigned>(i >> 31) + a + 0x85ebca6bU);
    float u1 = (static_cast<float>(a >> 8) + 1.0f) * (1.0f / 16777217.0f);
    float u2 = static_cast<float>(b >> 8) * (1.0f / 16777216.0f);
    float z = sqrtf(-2.0f * logf(u1)) * cosf(6.2831853f * u2);
    out[i] = static_cast<T>(mean + std * z);
  }
}

// The reference's weight map with its accessors answered from a table of device
// pointers (the reference does the same for GGUF models with its
// QuantizedWeightMapAdapter): LlamaForwardTyped reads weights only through these
// virtual functions and reinterprets the pointers as T (transformer_forward.cu:1760).
template <typename T> class TableWeights : public WeightMapTyped<half> {
public:
  struct Layer {
    T *q{}, *k{}, *v{}, *o{}, *in_norm{}, *post_norm{}, *gate{}, *up{}, *down{}, *qb{}, *kb{}, *vb{};
  };
  std::vector<Layer> layers;
  T *embed{}, *final_norm{}, *lm_head{};

  const half *LayerQProj(int l) const override { return h(layers[l].q); }
  const half *LayerKProj(int l) const override { return h(layers[l].k); }
  const half *LayerVProj(int l) const override { return h(layers[l].v); }
  const half *LayerOProj(int l) const override { return h(layers[l].o); }
  const half *LayerInputNorm(int l) const override { return h(layers[l].in_norm); }
  const half *LayerPostAttnNorm(int l) const override { return h(layers[l].post_norm); }
  const half *LayerGateProj(int l) const override { return h(layers[l].gate); }
  const half *LayerUpProj(int l) const override { return h(layers[l].up); }
  const half *LayerDownProj(int l) const override { return h(layers[l].down); }
  const half *LayerQProjBias(int l) const override { return h(layers[l].qb); }
  const half *LayerKProjBias(int l) const override { return h(layers[l].kb); }
  const half *LayerVProjBias(int l) const override { return h(layers[l].vb); }
  const half *EmbedTokens() const override { return h(embed); }
  const half *FinalNorm() const override { return h(final_norm); }
  const half *LmHead() const override { return h(lm_head ? lm_head : embed); }   // weight_map.cpp:33-37
  int NumLayers() const override { return static_cast<int>(layers.size()); }

private:
  static const half *h(const T *p) { return reinterpret_cast<const half *>(p); }
};

struct Shape {
  int hidden, layers, heads, kv_heads, head_dim, inter, vocab, max_pos;
  float theta, eps;
  bool tied, bias;
};

static Shape shape_from(const Args &a) {
  Shape s;
  s.hidden = static_cast<int>(a.need("hidden"));
  s.layers = static_cast<int>(a.need("layers"));
  s.heads = static_cast<int>(a.need("heads"));
  s.kv_heads = static_cast<int>(a.need("kv_heads"));
  s.head_dim = static_cast<int>(a.need("head_dim"));
  s.inter = static_cast<int>(a.need("inter"));
  s.vocab = static_cast<int>(a.need("vocab"));
  s.max_pos = static_cast<int>(a.num("max_pos", 4096));
  s.theta = static_cast<float>(a.real("theta", 10000.0));
  s.eps = static_cast<float>(a.real("eps", 1e-6));
  s.tied = a.num("tied", 0) != 0;
  s.bias = a.num("bias", 1) != 0;
  return s;
}

template <typename T> static T *device_random(size_t n, unsigned seed, float mean, float std) {
  T *d = nullptr;
  CK(cudaMalloc(&d, n * sizeof(T)));
  fill_normal_kernel<T><<<1184, 256>>>(d, n, seed, mean, std);
  CK(cudaGetLastError());
  return d;
}

// A tensor of the model: from `<dir>/<name>.bin` (raw T, as the caller wrote it) when a
// folder is given, else made up.
template <typename T>
static T *tensor(const std::string &dir, const std::string &name, size_t n, unsigned &seed, float mean,
                 float std, bool optional = false) {
  if (!dir.empty()) {
    const std::string path = dir + "/" + name + ".bin";
    if (!file_exists(path)) {
      if (optional) return nullptr;
      die("missing tensor file " + path);
    }
    auto bytes = read_file(path);
    if (bytes.size() != n * sizeof(T))
      die(path + " has " + std::to_string(bytes.size()) + " bytes, expected " + std::to_string(n * sizeof(T)));
    return upload<T>(bytes);
  }
  return device_random<T>(n, seed++, mean, std);
}

template <typename T> static std::unique_ptr<TableWeights<T>> make_weights(const Shape &s, const std::string &dir) {
  auto w = std::make_unique<TableWeights<T>>();
  unsigned seed = 1;
  const size_t H = s.hidden, Q = static_cast<size_t>(s.heads) * s.head_dim,
               KV = static_cast<size_t>(s.kv_heads) * s.head_dim, I = s.inter, V = s.vocab;
  w->embed = tensor<T>(dir, "model.embed_tokens.weight", V * H, seed, 0.f, 0.02f);
  w->final_norm = tensor<T>(dir, "model.norm.weight", H, seed, 1.f, 0.f);
  w->lm_head = s.tied ? nullptr : tensor<T>(dir, "lm_head.weight", V * H, seed, 0.f, 0.02f);
  w->layers.resize(s.layers);
  for (int l = 0; l < s.layers; ++l) {
    const std::string p = "model.layers." + std::to_string(l) + ".";
    auto &L = w->layers[l];
    L.in_norm = tensor<T>(dir, p + "input_layernorm.weight", H, seed, 1.f, 0.f);
    L.post_norm = tensor<T>(dir, p + "post_attention_layernorm.weight", H, seed, 1.f, 0.f);
    L.q = tensor<T>(dir, p + "self_attn.q_proj.weight", Q * H, seed, 0.f, 0.02f);
    L.k = tensor<T>(dir, p + "self_attn.k_proj.weight", KV * H, seed, 0.f, 0.02f);
    L.v = tensor<T>(dir, p + "self_attn.v_proj.weight", KV * H, seed, 0.f, 0.02f);
    L.o = tensor<T>(dir, p + "self_attn.o_proj.weight", H * Q, seed, 0.f, 0.02f);
    if (s.bias) {
      L.qb = tensor<T>(dir, p + "self_attn.q_proj.bias", Q, seed, 0.f, 0.02f, true);
      L.kb = tensor<T>(dir, p + "self_attn.k_proj.bias", KV, seed, 0.f, 0.02f, true);
      L.vb = tensor<T>(dir, p + "self_attn.v_proj.bias", KV, seed, 0.f, 0.02f, true);
    }
    L.gate = tensor<T>(dir, p + "mlp.gate_proj.weight", I * H, seed, 0.f, 0.02f);
    L.up = tensor<T>(dir, p + "mlp.up_proj.weight", I * H, seed, 0.f, 0.02f);
    L.down = tensor<T>(dir, p + "mlp.down_proj.weight", H * I, seed, 0.f, 0.02f);
  }
  CK(cudaDeviceSynchronize());
  return w;
}

// Everything the reference needs to run its dense model, built the way
// InferfluxCudaExecutor does (runtime/backends/cuda/inferflux_cuda_executor.cpp:1943-1972):
// typed forward from the factory, policy from the environment, prefill chunk cap,
// Initialize, WarmWeightCaches.
template <typename T> struct RefModel {
  Shape shape;
  std::unique_ptr<TableWeights<T>> weights;
  std::unique_ptr<KvCacheGpuTyped<T>> cache;
  std::unique_ptr<CublasGemm> gemm;
  std::unique_ptr<ModelForward> forward;
  std::unique_ptr<GpuSampler> sampler;
  cudaStream_t stream{};
  float *d_logits{};

  void build(const Shape &s, const std::string &weight_dir, int max_seq, int max_batch, int chunk) {
    shape = s;
    CK(cudaStreamCreate(&stream));
    weights = make_weights<T>(s, weight_dir);
    cache = std::make_unique<KvCacheGpuTyped<T>>();
    if (!cache->Allocate(s.layers, s.kv_heads, s.head_dim, max_seq, max_batch)) die("KV cache allocation failed");
    gemm = std::make_unique<CublasGemm>();
    if (!gemm->Initialize(stream)) die("cuBLAS initialisation failed");
    SafetensorsLoader::ModelConfig cfg;
    cfg.hidden_size = s.hidden;
    cfg.num_hidden_layers = s.layers;
    cfg.num_attention_heads = s.heads;
    cfg.num_key_value_heads = s.kv_heads;
    cfg.head_dim = s.head_dim;
    cfg.intermediate_size = s.inter;
    cfg.vocab_size = s.vocab;
    cfg.max_position_embeddings = s.max_pos;
    cfg.rope_freq_base = s.theta;
    cfg.model_type = "qwen2";
    cfg.activation = "silu";
    cfg.torch_dtype = std::is_same<T, __nv_bfloat16>::value ? "bfloat16" : "float16";
    cfg.rms_norm_eps = s.eps;
    forward = CreateModelForwardTyped<T>(cfg.model_type);
    if (!forward) die("the reference's factory knows no model_type qwen2");
    forward->SetExecutionPolicy(NativeExecutionPolicy::FromEnv());
    forward->SetPrefillChunkTokens(chunk);
    if (!forward->Initialize(cfg, *weights, cache.get(), gemm.get(), stream)) die("ModelForward::Initialize failed");
    forward->WarmWeightCaches();
    sampler = std::make_unique<GpuSampler>();
    if (!sampler->Initialize(s.vocab, stream)) die("GpuSampler::Initialize failed");
    CK(cudaMalloc(&d_logits, static_cast<size_t>(max_batch) * s.vocab * sizeof(float)));
    CK(cudaDeviceSynchronize());
  }
};

// ----------------------------------------------------------------------- bench
static std::vector<int> random_tokens(int n, int vocab, unsigned seed) {
  std::vector<int> t(n);
  unsigned x = seed * 2654435761u + 12345u;
  for (int i = 0; i < n; ++i) {
    x = x * 1664525u + 1013904223u;
    t[i] = static_cast<int>((x >> 8) % static_cast<unsigned>(vocab));
  }
  return t;
}

// Bring sequence 0 to `length` tokens with Forward calls of at most `chunk` tokens, then give
// the other `batch - 1` sequences the same prefix with the cache's own prefix copy.
template <typename T>
static void fill_sequences(RefModel<T> &m, int batch, int length, int chunk, unsigned seed) {
  auto toks = random_tokens(length, m.shape.vocab, seed);
  for (int at = 0; at < length; at += chunk) {
    int n = std::min(chunk, length - at);
    std::vector<int> part(toks.begin() + at, toks.begin() + at + n);
    if (!m.forward->Forward(part, at, 0, m.d_logits)) die("Forward failed while filling the cache");
  }
  for (int b = 1; b < batch; ++b)
    if (!m.cache->CopySequencePrefix(0, b, length, m.stream)) die("CopySequencePrefix failed");
  CK(cudaStreamSynchronize(m.stream));
}

template <typename T> static int bench(const Args &a) {
  const Shape s = shape_from(a);
  const std::vector<int> batches = ints(a.str("batches", "8"));
  const int steps = static_cast<int>(a.num("steps", 20)), warmup = static_cast<int>(a.num("warmup", 5));
  const int ctx_end = static_cast<int>(a.num("ctx_end", 4096));
  const int prefill_tokens = static_cast<int>(a.num("prefill_tokens", 2048));
  const int prefill_reps = static_cast<int>(a.num("prefill_reps", 5));
  int max_batch = 1;
  for (int b : batches) max_batch = std::max(max_batch, b);
  RefModel<T> m;
  m.build(s, "", ctx_end, max_batch, std::max(prefill_tokens, 1));
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  std::printf("{\"ok\": 1");

  // ---- one prompt of `prefill_tokens` tokens in one Forward call
  if (prefill_tokens > 0) {
    std::vector<float> ms;
    for (int i = 0; i < 3 + prefill_reps; ++i) {
      auto toks = random_tokens(prefill_tokens, s.vocab, 100 + i);
      CK(cudaStreamSynchronize(m.stream));
      CK(cudaEventRecord(e0, m.stream));
      if (!m.forward->Forward(toks, 0, 0, m.d_logits)) die("Forward (prefill) failed");
      CK(cudaEventRecord(e1, m.stream));
      CK(cudaStreamSynchronize(m.stream));
      float t = 0;
      CK(cudaEventElapsedTime(&t, e0, e1));
      if (i >= 3) ms.push_back(t);
    }
    std::sort(ms.begin(), ms.end());
    std::printf(", \"prefill_ms\": %.4f, \"prefill_tokens\": %d", ms[ms.size() / 2], prefill_tokens);
  }

  // ---- decode: one token of each of B sequences per step
  for (int B : batches) {
    const int total = 2 * (warmup + steps);
    const int start = ctx_end - total;
    if (start < 1) die("ctx_end leaves no room for the decode steps");
    fill_sequences(m, B, start, std::max(prefill_tokens, 1), 7u + B);
    std::vector<int> seqs(B), n_past(B, start), toks = random_tokens(B, s.vocab, 9u + B), out;
    for (int b = 0; b < B; ++b) seqs[b] = b;
    const std::vector<float> temps(B, 0.0f), top_ps(B, 1.0f);
    const std::vector<int> top_ks(B, 0);
    const std::vector<uint32_t> seeds(B, UINT32_MAX);

    // end to end: host token ids in, sampled ids back on the host, every step
    double t_begin = 0, wall0 = 0;
    for (int i = 0; i < warmup + steps; ++i) {
      if (i == warmup) {
        CK(cudaStreamSynchronize(m.stream));
        t_begin = now_unix();
        wall0 = t_begin;
      }
      if (!m.forward->BatchForward(toks, n_past, seqs, m.d_logits, B)) die("BatchForward failed");
      m.sampler->SampleBatch(m.d_logits, B, temps, top_ks, top_ps, seeds, &out);
      for (int b = 0; b < B; ++b) {
        toks[b] = out[b];
        n_past[b] += 1;
      }
    }
    CK(cudaStreamSynchronize(m.stream));
    const double e2e_ms = (now_unix() - wall0) * 1000.0 / steps;

    // on the device: the same calls without reading the ids back, timed with events
    auto feed = random_tokens(B * (warmup + steps), s.vocab, 31u + B);
    double d_begin = 0, d_end = 0;
    for (int i = 0; i < warmup + steps; ++i) {
      if (i == warmup) {
        CK(cudaStreamSynchronize(m.stream));
        d_begin = now_unix();
        CK(cudaEventRecord(e0, m.stream));
      }
      std::vector<int> t(feed.begin() + i * B, feed.begin() + (i + 1) * B);
      if (!m.forward->BatchForward(t, n_past, seqs, m.d_logits, B)) die("BatchForward failed");
      if (!m.sampler->EnqueueBatchedArgmax(m.d_logits, B)) die("EnqueueBatchedArgmax failed");
      for (int b = 0; b < B; ++b) n_past[b] += 1;
    }
    CK(cudaEventRecord(e1, m.stream));
    CK(cudaStreamSynchronize(m.stream));
    d_end = now_unix();
    float dev = 0;
    CK(cudaEventElapsedTime(&dev, e0, e1));
    std::printf(", \"b%d\": {\"dev_ms\": %.5f, \"e2e_ms\": %.5f, \"ctx_end\": %d, \"timed_begin\": %.3f, "
                "\"timed_end\": %.3f, \"graph\": %d, \"h2d_bytes\": %d, \"d2h_bytes\": %d}",
                B, dev / steps, e2e_ms, n_past[0], d_begin, d_end, m.forward->DecodeGraphReady(B) ? 1 : 0,
                m.forward->GetMaxBatchSize() * 16, B * 4);
    (void)t_begin;
  }
  std::printf("}\n");
  std::fflush(stdout);
  return 0;
}

// ----------------------------------------------------------------------- model
// Runs a script of calls on a model whose weights lie as raw files in `weights=`:
//   forward seq=S n_past=P tokens=1,2,3 out=FILE      logits of the last token, float32 [vocab]
//   batch tokens=5,6 n_past=3,7 seqs=0,1 out=FILE     float32 [B, vocab]
template <typename T> static int model(const Args &a) {
  const Shape s = shape_from(a);
  RefModel<T> m;
  m.build(s, a.str("weights"), static_cast<int>(a.num("max_seq", 256)), static_cast<int>(a.num("max_batch", 4)),
          static_cast<int>(a.num("chunk", 256)));
  std::ifstream script(a.str("script"));
  if (!script) die("cannot read script " + a.str("script"));
  const std::string out_dir = a.str("out", ".");
  std::string line;
  while (std::getline(script, line)) {
    if (line.empty() || line[0] == '#') continue;
    std::stringstream ss(line);
    std::string cmd, kvs;
    ss >> cmd;
    Args c;
    while (ss >> kvs) {
      auto eq = kvs.find('=');
      if (eq == std::string::npos) die("script: expected key=value in: " + line);
      c.kv[kvs.substr(0, eq)] = kvs.substr(eq + 1);
    }
    if (cmd == "forward") {
      auto toks = ints(c.str("tokens"));
      if (!m.forward->Forward(toks, static_cast<int>(c.need("n_past")), static_cast<int>(c.need("seq")), m.d_logits))
        die("Forward failed: " + line);
      CK(cudaStreamSynchronize(m.stream));
      download_to<float>(out_dir + "/" + c.str("out"), m.d_logits, s.vocab);
    } else if (cmd == "batch") {
      auto toks = ints(c.str("tokens")), past = ints(c.str("n_past")), seqs = ints(c.str("seqs"));
      const int B = static_cast<int>(toks.size());
      if (static_cast<int>(past.size()) != B || static_cast<int>(seqs.size()) != B) die("script: batch lists differ: " + line);
      if (!m.forward->BatchForward(toks, past, seqs, m.d_logits, B)) die("BatchForward failed: " + line);
      CK(cudaStreamSynchronize(m.stream));
      download_to<float>(out_dir + "/" + c.str("out"), m.d_logits, static_cast<size_t>(B) * s.vocab);
    } else {
      die("script: unknown command " + cmd);
    }
  }
  std::printf("{\"ok\": 1}\n");
  return 0;
}

// ------------------------------------------------------------------------ leaf
// One host wrapper of the reference on inputs read from `dir=`; outputs go there too.
template <typename T> static T *in(const Args &a, const std::string &name, size_t n) {
  auto bytes = read_file(a.str("dir") + "/" + name + ".bin");
  if (bytes.size() != n * sizeof(T)) die(name + ".bin has the wrong size");
  return upload<T>(bytes);
}

template <typename T> static int leaf(const Args &a) {
  const std::string op = a.str("op"), dir = a.str("dir");
  cudaStream_t st = nullptr;
  if (op == "rmsnorm") {                       // cuda_kernels.cu:16-47
    const int rows = a.need("rows"), H = a.need("hidden");
    T *x = in<T>(a, "x", size_t(rows) * H), *w = in<T>(a, "w", H), *y;
    CK(cudaMalloc(&y, size_t(rows) * H * sizeof(T)));
    CK(cuda_kernel::RmsNorm<T>(x, w, y, rows, H, float(a.real("eps", 1e-6)), st));
    CK(cudaDeviceSynchronize());
    download_to<T>(dir + "/y.bin", y, size_t(rows) * H);
  } else if (op == "add_rmsnorm_mixed") {      // cuda_kernels.cu:618-655
    const int rows = a.need("rows"), H = a.need("hidden");
    float *res = in<float>(a, "residual", size_t(rows) * H);
    T *x = in<T>(a, "x", size_t(rows) * H), *w = in<T>(a, "w", H), *y;
    CK(cudaMalloc(&y, size_t(rows) * H * sizeof(T)));
    CK(cuda_kernel::ResidualAddRmsNormMixed<T>(res, x, w, y, rows, H, float(a.real("eps", 1e-6)), st));
    CK(cudaDeviceSynchronize());
    download_to<T>(dir + "/y.bin", y, size_t(rows) * H);
    download_to<float>(dir + "/residual_out.bin", res, size_t(rows) * H);
  } else if (op == "rope") {                   // cuda_kernels.cu:93-116, rope_type 2 = split-half
    const int T_ = a.need("seq_len"), nh = a.need("heads"), nkv = a.need("kv_heads"), d = a.need("head_dim");
    T *q = in<T>(a, "q", size_t(T_) * nh * d), *k = in<T>(a, "k", size_t(T_) * nkv * d);
    CK(cuda_kernel::RoPE<T>(q, k, T_, nh, nkv, d, int(a.need("n_past")), float(a.real("theta", 10000.0)), st,
                            int(a.num("rope_type", 2))));
    CK(cudaDeviceSynchronize());
    download_to<T>(dir + "/q_out.bin", q, size_t(T_) * nh * d);
    download_to<T>(dir + "/k_out.bin", k, size_t(T_) * nkv * d);
  } else if (op == "batched_rope") {           // cuda_kernels.cu:895-958: bias folded in before the rotation
    const int B = a.need("batch"), nh = a.need("heads"), nkv = a.need("kv_heads"), d = a.need("head_dim");
    T *q = in<T>(a, "q", size_t(B) * nh * d), *k = in<T>(a, "k", size_t(B) * nkv * d);
    T *qb = a.num("bias", 0) ? in<T>(a, "q_bias", size_t(nh) * d) : nullptr;
    T *kb = a.num("bias", 0) ? in<T>(a, "k_bias", size_t(nkv) * d) : nullptr;
    int *past = in<int>(a, "n_past", B);
    CK(cuda_kernel::BatchedRoPE<T>(q, k, B, nh, nkv, d, past, float(a.real("theta", 10000.0)), st,
                                   int(a.num("rope_type", 2)), qb, kb));
    CK(cudaDeviceSynchronize());
    download_to<T>(dir + "/q_out.bin", q, size_t(B) * nh * d);
    download_to<T>(dir + "/k_out.bin", k, size_t(B) * nkv * d);
  } else if (op == "silu_mul") {               // cuda_kernels.cu:147-150
    const int n = a.need("count");
    T *g = in<T>(a, "gate", n), *u = in<T>(a, "up", n), *y;
    CK(cudaMalloc(&y, size_t(n) * sizeof(T)));
    CK(cuda_kernel::SiluMul<T>(g, u, y, n, st));
    CK(cudaDeviceSynchronize());
    download_to<T>(dir + "/y.bin", y, n);
  } else if (op == "bias_triple") {            // cuda_kernels.cu:777-804
    const int rows = a.need("rows"), qd = a.need("q_dim"), kd = a.need("k_dim");
    T *q = in<T>(a, "q", size_t(rows) * qd), *k = in<T>(a, "k", size_t(rows) * kd), *v = in<T>(a, "v", size_t(rows) * kd);
    T *qb = in<T>(a, "q_bias", qd), *kb = in<T>(a, "k_bias", kd), *vb = in<T>(a, "v_bias", kd);
    CK(cuda_kernel::BiasAddTriple<T>(q, k, v, qb, kb, vb, rows, qd, kd, kd, st));
    CK(cudaDeviceSynchronize());
    download_to<T>(dir + "/q_out.bin", q, size_t(rows) * qd);
    download_to<T>(dir + "/k_out.bin", k, size_t(rows) * kd);
    download_to<T>(dir + "/v_out.bin", v, size_t(rows) * kd);
  } else if (op == "attn_prefill") {           // flash_attention.cu:422-456; K/V are [kv_len, kv_heads * head_dim]
    const int ql = a.need("query_len"), kl = a.need("kv_len"), nh = a.need("heads"), nkv = a.need("kv_heads"),
              d = a.need("head_dim");
    T *q = in<T>(a, "q", size_t(ql) * nh * d), *k = in<T>(a, "k", size_t(kl) * nkv * d),
      *v = in<T>(a, "v", size_t(kl) * nkv * d), *o;
    CK(cudaMalloc(&o, size_t(ql) * nh * d * sizeof(T)));
    CK(cuda_kernel::FlashAttention2Typed<T>(q, k, v, o, 1, ql, kl, nh, nkv, d, 1.0f / sqrtf(float(d)), true, st));
    CK(cudaDeviceSynchronize());
    download_to<T>(dir + "/o.bin", o, size_t(ql) * nh * d);
  } else if (op == "attn_decode") {            // flash_attention.cu:2118-2135; cache [slots][layers][2][max_seq][kv_dim]
    const int B = a.need("batch"), nh = a.need("heads"), nkv = a.need("kv_heads"), d = a.need("head_dim"),
              max_seq = a.need("max_seq"), slots = a.need("slots");
    const size_t kv_dim = size_t(nkv) * d, kv_stride = size_t(max_seq) * kv_dim, layer_stride = 2 * kv_stride,
                 slot_stride = layer_stride;                      // one layer
    T *q = in<T>(a, "q", size_t(B) * nh * d), *cache = in<T>(a, "cache", size_t(slots) * slot_stride), *o;
    int *seq_ids = in<int>(a, "seq_ids", B), *kv_lens = in<int>(a, "kv_lens", B);
    CK(cudaMalloc(&o, size_t(B) * nh * d * sizeof(T)));
    CK(cuda_kernel::FlashDecodeMultiSeqStrided<T>(q, cache, o, seq_ids, kv_lens, 0, B, nh, nkv, d, slot_stride,
                                                  layer_stride, kv_stride, 1.0f / sqrtf(float(d)), st));
    CK(cudaDeviceSynchronize());
    download_to<T>(dir + "/o.bin", o, size_t(B) * nh * d);
  } else {
    die("leaf: unknown op " + op);
  }
  std::printf("{\"ok\": 1}\n");
  return 0;
}

int main(int argc, char **argv) {
  if (argc < 2) die("usage: ref_harness bench|model|leaf key=value ...");
  const std::string mode(argv[1]);
  const Args a = parse(argc, argv, 2);
  const bool f16 = a.str("dtype", "bf16") == "f16";
  CK(cudaSetDevice(0));
  if (mode == "bench") return f16 ? bench<half>(a) : bench<__nv_bfloat16>(a);
  if (mode == "model") return f16 ? model<half>(a) : model<__nv_bfloat16>(a);
  if (mode == "leaf") return f16 ? leaf<half>(a) : leaf<__nv_bfloat16>(a);
  die("unknown mode " + mode);
  return 2;
}
