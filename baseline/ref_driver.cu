// Host driver for the UNMODIFIED reference (AlterHoodie/poor_mans_mamba, "MambaServe") CUDA path.
//
// It links the reference's own translation units (src/ops/gpu/*.cu, src/ops/cuda_backend.cu,
// src/core/{device.cpp,cuda_allocator.cu}, src/runtime/cache/{cache_layout,cache_pool}.cpp,
// src/runtime/runner/falconh1_runner.cpp) and drives FalconH1Runner::prefill / ::decode
// (src/runtime/runner/falconh1_runner.cpp:216-248) through CUDABackend, the stock code path.
// Nothing of the engine in this repository is on that path.  What this file adds is only what the
// reference takes from libraries that cannot be had offline: reading config.json (nlohmann_json
// there) and model.safetensors (safetensors-cpp there), by the key names of
// src/io/config_parser.cpp:95-162 and src/model/falconh1_loader.cpp:27-58, with the dtype rule of
// src/io/model_loader.cpp:78-99 (F32 copied, BF16 widened, everything FP32 on the device).
//
//   ref_driver logits --model DIR --max-seq N --tokens a,b,c --decode x,y,z --out FILE
//       prefill the tokens in one call, then feed the decode tokens one by one; FILE receives
//       [1 + n_decode, vocab] little-endian float32 logits (last position of the prefill, then one
//       row per decoded token).
//   ref_driver bench --config DIR --batch B --context C --steps K --warmup W [--prefill-len T]
//       random weights made on the device (the reference has no random-weights mode; its tests fill
//       constants by hand, tests/runtime/runner/falconh1runner_test.cpp:86-137).  Batch 1 is timed
//       the way benchmarks/generate_bench.cpp:228-255 and :329-367 do (ExecContext{}, a device
//       synchronize and a host argmax per token); batch B > 1 is B cache slots on B streams with a
//       cuBLAS handle each, as src/runtime/worker.cpp:121-142 sets them up.  Prints one JSON object.
#include <cublas_v2.h>
#include <cuda_runtime.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <string>
#include <vector>

#include "core/device.h"
#include "io/config.h"
#include "model/falconh1_weights.h"
#include "ops/backend.h"
#include "ops/common/tensor_checks.h"
#include "runtime/cache/cache_layout.h"
#include "runtime/cache/cache_pool.h"
#include "runtime/runner/falconh1_runner.h"

namespace {

[[noreturn]] void die(const std::string& msg) {
  std::fprintf(stderr, "ref_driver: %s\n", msg.c_str());
  std::exit(1);
}

#define CUDA_OK(call)                                                                              \
  do {                                                                                             \
    cudaError_t e_ = (call);                                                                       \
    if (e_ != cudaSuccess)                                                                         \
      die(std::string(#call) + ": " + cudaGetErrorString(e_));                                     \
  } while (0)

// ---------------------------------------------------------------------------------------------
// A small JSON reader (objects, arrays, strings, numbers, true/false/null).
// ---------------------------------------------------------------------------------------------
struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;

  const Json* find(const std::string& k) const {
    for (const auto& kv : obj)
      if (kv.first == k)
        return &kv.second;
    return nullptr;
  }
};

struct JsonParser {
  const char* p;
  const char* end;
  void ws() {
    while (p < end && (*p == ' ' || *p == '\n' || *p == '\t' || *p == '\r'))
      ++p;
  }
  Json parse() {
    ws();
    if (p >= end)
      die("json: unexpected end");
    Json v;
    if (*p == '{') {
      v.kind = Json::Obj;
      ++p;
      ws();
      if (*p == '}') {
        ++p;
        return v;
      }
      while (true) {
        ws();
        Json k = parse();
        if (k.kind != Json::Str)
          die("json: object key must be a string");
        ws();
        if (*p != ':')
          die("json: ':' expected");
        ++p;
        v.obj.emplace_back(k.str, parse());
        ws();
        if (*p == ',') {
          ++p;
          continue;
        }
        if (*p == '}') {
          ++p;
          return v;
        }
        die("json: ',' or '}' expected");
      }
    }
    if (*p == '[') {
      v.kind = Json::Arr;
      ++p;
      ws();
      if (*p == ']') {
        ++p;
        return v;
      }
      while (true) {
        v.arr.push_back(parse());
        ws();
        if (*p == ',') {
          ++p;
          continue;
        }
        if (*p == ']') {
          ++p;
          return v;
        }
        die("json: ',' or ']' expected");
      }
    }
    if (*p == '"') {
      v.kind = Json::Str;
      ++p;
      while (p < end && *p != '"') {
        if (*p == '\\' && p + 1 < end) {
          ++p;
          switch (*p) {
          case 'n': v.str.push_back('\n'); break;
          case 't': v.str.push_back('\t'); break;
          case 'u': p += 4; v.str.push_back('?'); break;
          default: v.str.push_back(*p);
          }
          ++p;
        } else {
          v.str.push_back(*p++);
        }
      }
      ++p;
      return v;
    }
    if (!std::strncmp(p, "true", 4)) {
      v.kind = Json::Bool;
      v.b = true;
      p += 4;
      return v;
    }
    if (!std::strncmp(p, "false", 5)) {
      v.kind = Json::Bool;
      p += 5;
      return v;
    }
    if (!std::strncmp(p, "null", 4)) {
      p += 4;
      return v;
    }
    char* q = nullptr;
    v.kind = Json::Num;
    v.num = std::strtod(p, &q);
    if (q == p)
      die("json: bad token");
    p = q;
    return v;
  }
};

Json parse_json(const char* data, size_t n) {
  JsonParser jp{data, data + n};
  return jp.parse();
}

double need_num(const Json& j, const char* key) {
  const Json* v = j.find(key);
  if (!v || v->kind != Json::Num)
    die(std::string("config field '") + key + "': missing or not a number");
  return v->num;
}
double opt_num(const Json& j, const char* key, double dflt) {
  const Json* v = j.find(key);
  return (v && v->kind == Json::Num) ? v->num : dflt;
}
bool opt_bool(const Json& j, const char* key, bool dflt) {
  const Json* v = j.find(key);
  return (v && v->kind == Json::Bool) ? v->b : dflt;
}

// config.json -> ModelConfig, key for key as src/io/config_parser.cpp:95-162 reads them.
ModelConfig read_config(const std::string& dir, int max_seq) {
  std::ifstream fh(dir + "/config.json");
  if (!fh)
    die("cannot open " + dir + "/config.json");
  std::stringstream ss;
  ss << fh.rdbuf();
  const std::string text = ss.str();
  Json j = parse_json(text.data(), text.size());

  ModelConfig cfg{};
  cfg.layout = ArchLayout::ParallelHybrid;
  cfg.model_type = "falcon_h1";
  const Json* mt = j.find("model_type");
  if (!mt || mt->str != "falcon_h1")
    die("expected model_type falcon_h1");
  cfg.hidden_size = static_cast<int>(need_num(j, "hidden_size"));
  cfg.vocab_size = static_cast<int>(need_num(j, "vocab_size"));
  cfg.tie_word_embeddings = opt_bool(j, "tie_word_embeddings", false);
  cfg.num_hidden_layers = static_cast<int>(need_num(j, "num_hidden_layers"));
  cfg.max_seq_length = max_seq;
  cfg.bos_token_id = static_cast<int>(opt_num(j, "bos_token_id", 0));
  cfg.eos_token_id = static_cast<int>(opt_num(j, "eos_token_id", -1));
  cfg.pad_token_id = static_cast<int>(opt_num(j, "pad_token_id", 0));
  cfg.rms_norm_eps = static_cast<float>(opt_num(j, "rms_norm_eps", 1e-5));

  AttnConfig attn{};
  attn.n_q_heads = static_cast<int>(need_num(j, "num_attention_heads"));
  attn.n_kv_heads = static_cast<int>(need_num(j, "num_key_value_heads"));
  attn.head_dim = static_cast<int>(need_num(j, "head_dim"));
  attn.rope_theta = static_cast<float>(opt_num(j, "rope_theta", 10000.0));
  cfg.attn = attn;

  cfg.ssm.n_heads = static_cast<int>(need_num(j, "mamba_n_heads"));
  cfg.ssm.d_head = static_cast<int>(need_num(j, "mamba_d_head"));
  cfg.ssm.d_state = static_cast<int>(need_num(j, "mamba_d_state"));
  cfg.ssm.d_conv = static_cast<int>(need_num(j, "mamba_d_conv"));
  cfg.ssm.d_inner = static_cast<int>(need_num(j, "mamba_d_ssm"));
  cfg.ssm.n_groups = static_cast<int>(need_num(j, "mamba_n_groups"));
  cfg.ssm.chunk_size = static_cast<int>(opt_num(j, "mamba_chunk_size", 128));
  cfg.ssm.use_conv_bias = opt_bool(j, "mamba_conv_bias", true);
  cfg.ssm.use_proj_bias = opt_bool(j, "mamba_proj_bias", false);
  cfg.ssm.gated_rms_norm = opt_bool(j, "mamba_rms_norm", false);

  ScaleConfig sc{};
  if (const Json* m = j.find("ssm_multipliers")) {
    if (m->arr.size() != 5)
      die("ssm_multipliers must have length 5 [z,x,B,C,dt]");
    for (size_t i = 0; i < 5; ++i)
      sc.ssm_chunk[i] = static_cast<float>(m->arr[i].num);
  }
  if (const Json* m = j.find("mlp_multipliers")) {
    if (m->arr.size() != 2)
      die("mlp_multipliers must have length 2");
    sc.mlp[0] = static_cast<float>(m->arr[0].num);
    sc.mlp[1] = static_cast<float>(m->arr[1].num);
  }
  sc.ssm_in = static_cast<float>(opt_num(j, "ssm_in_multiplier", 1.0));
  sc.ssm_out = static_cast<float>(opt_num(j, "ssm_out_multiplier", 1.0));
  sc.attn_in = static_cast<float>(opt_num(j, "attention_in_multiplier", 1.0));
  sc.attn_out = static_cast<float>(opt_num(j, "attention_out_multiplier", 1.0));
  sc.key = static_cast<float>(opt_num(j, "key_multiplier", 1.0));
  sc.embedding = static_cast<float>(opt_num(j, "embedding_multiplier", 1.0));
  sc.lm_head = static_cast<float>(opt_num(j, "lm_head_multiplier", 1.0));
  cfg.scales = sc;

  MlpConfig mlp{};
  mlp.intermediate_size = static_cast<int>(need_num(j, "intermediate_size"));
  cfg.mlp = mlp;
  return cfg;
}

// ---------------------------------------------------------------------------------------------
// Tensors on the device, through the reference's allocator (the caller holds an AllocatorScope).
// ---------------------------------------------------------------------------------------------
Tensor device_tensor(std::vector<int64_t> shape) {
  StatusOr<Tensor> t = allocate_f32_tensor(std::move(shape));
  if (!t.ok())
    die("allocate_f32_tensor: " + t.status().message());
  return std::move(t.value());
}

Tensor upload(const std::vector<float>& host, std::vector<int64_t> shape) {
  Tensor t = device_tensor(std::move(shape));
  if (t.buffer.bytes != host.size() * sizeof(float))
    die("upload: size mismatch");
  CUDA_OK(cudaMemcpy(t.buffer.ptr, host.data(), t.buffer.bytes, cudaMemcpyHostToDevice));
  return t;
}

struct SafeTensors {
  const uint8_t* base = nullptr;
  size_t bytes = 0;
  const uint8_t* data = nullptr;
  Json header;

  explicit SafeTensors(const std::string& path) {
    int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0)
      die("cannot open " + path);
    struct stat st {};
    if (::fstat(fd, &st) != 0)
      die("cannot stat " + path);
    bytes = static_cast<size_t>(st.st_size);
    void* m = ::mmap(nullptr, bytes, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED)
      die("mmap failed for " + path);
    base = static_cast<const uint8_t*>(m);
    uint64_t hlen = 0;
    std::memcpy(&hlen, base, 8);
    if (8 + hlen > bytes)
      die("safetensors header longer than the file");
    header = parse_json(reinterpret_cast<const char*>(base + 8), hlen);
    data = base + 8 + hlen;
  }

  // F32 copied, BF16 widened, anything else refused (src/io/model_loader.cpp:78-99).
  Tensor load(const std::string& name, std::vector<int64_t> shape) const {
    const Json* e = header.find(name);
    if (!e)
      die("missing tensor: " + name);
    const Json* dt = e->find("dtype");
    const Json* sh = e->find("shape");
    const Json* off = e->find("data_offsets");
    if (!dt || !sh || !off || off->arr.size() != 2)
      die("malformed safetensors entry: " + name);
    int64_t numel = 1;
    for (const Json& d : sh->arr)
      numel *= static_cast<int64_t>(d.num);
    int64_t want = 1;
    for (int64_t d : shape)
      want *= d;
    if (numel != want)
      die("tensor " + name + ": element count does not match the configuration");
    const uint8_t* src = data + static_cast<size_t>(off->arr[0].num);
    std::vector<float> host(static_cast<size_t>(numel));
    if (dt->str == "F32") {
      std::memcpy(host.data(), src, host.size() * 4);
    } else if (dt->str == "BF16") {
      const uint16_t* h = reinterpret_cast<const uint16_t*>(src);
      for (int64_t i = 0; i < numel; ++i) {
        uint32_t bits = static_cast<uint32_t>(h[i]) << 16;
        std::memcpy(&host[static_cast<size_t>(i)], &bits, 4);
      }
    } else {
      die("expected F32 or BF16 for tensor: " + name);
    }
    return upload(host, std::move(shape));
  }
};

struct Dims {
  int64_t D, V, F, I, G, N, H, K, conv_dim, proj, q_dim, kv_dim;
};

Dims dims_of(const ModelConfig& c) {
  Dims d{};
  d.D = c.hidden_size;
  d.V = c.vocab_size;
  d.F = c.mlp->intermediate_size;
  d.I = c.ssm.d_inner;
  d.G = c.ssm.n_groups;
  d.N = c.ssm.d_state;
  d.H = c.ssm.n_heads;
  d.K = c.ssm.d_conv;
  d.conv_dim = d.I + 2 * d.G * d.N;
  d.proj = d.I + d.conv_dim + d.H;
  d.q_dim = static_cast<int64_t>(c.attn->n_q_heads) * c.attn->head_dim;
  d.kv_dim = static_cast<int64_t>(c.attn->n_kv_heads) * c.attn->head_dim;
  return d;
}

// Tensor names of src/model/falconh1_loader.cpp:27-58.
FalconH1Weights load_weights(const ModelConfig& cfg, const std::string& dir) {
  SafeTensors st(dir + "/model.safetensors");
  const Dims d = dims_of(cfg);
  FalconH1Weights w;
  w.embeddings = st.load("model.embed_tokens.weight", {d.V, d.D});
  w.norm_f = st.load("model.final_layernorm.weight", {d.D});
  if (!cfg.tie_word_embeddings)
    w.lm_head = st.load("lm_head.weight", {d.V, d.D});
  w.layers.resize(static_cast<size_t>(cfg.num_hidden_layers));
  for (int i = 0; i < cfg.num_hidden_layers; ++i) {
    FalconH1LayerWeights& L = w.layers[static_cast<size_t>(i)];
    const std::string p = "model.layers." + std::to_string(i);
    L.ff_up_proj = st.load(p + ".feed_forward.up_proj.weight", {d.F, d.D});
    L.ff_gate_proj = st.load(p + ".feed_forward.gate_proj.weight", {d.F, d.D});
    L.ff_down_proj = st.load(p + ".feed_forward.down_proj.weight", {d.D, d.F});
    L.A_log = st.load(p + ".mamba.A_log", {d.H});
    L.conv1d = st.load(p + ".mamba.conv1d.weight", {d.conv_dim, d.K});
    L.conv1d_bias = st.load(p + ".mamba.conv1d.bias", {d.conv_dim});
    L.D = st.load(p + ".mamba.D", {d.H});
    L.dt_bias = st.load(p + ".mamba.dt_bias", {d.H});
    L.in_proj = st.load(p + ".mamba.in_proj.weight", {d.proj, d.D});
    L.out_proj = st.load(p + ".mamba.out_proj.weight", {d.D, d.I});
    L.input_layernorm = st.load(p + ".input_layernorm.weight", {d.D});
    L.pre_ff_layer_norm = st.load(p + ".pre_ff_layernorm.weight", {d.D});
    L.q_proj = st.load(p + ".self_attn.q_proj.weight", {d.q_dim, d.D});
    L.k_proj = st.load(p + ".self_attn.k_proj.weight", {d.kv_dim, d.D});
    L.v_proj = st.load(p + ".self_attn.v_proj.weight", {d.kv_dim, d.D});
    L.o_proj = st.load(p + ".self_attn.o_proj.weight", {d.D, d.q_dim});
  }
  return w;
}

// Random weights for timing only, made on the device: matrices ~N(0, 0.02), A_log = log U[1,16],
// dt_bias = inverse softplus of a log-uniform step in [1e-3, 0.1], D = 1, norm weights 1.
__device__ inline uint32_t mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352dU;
  x ^= x >> 15;
  x *= 0x846ca68bU;
  x ^= x >> 16;
  return x;
}
__global__ void fill_normal(float* out, size_t n, uint32_t seed, float std_dev) {
  size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= n)
    return;
  uint32_t a = mix32(static_cast<uint32_t>(i) * 2654435761U + seed);
  uint32_t b = mix32(a ^ 0x9e3779b9U ^ static_cast<uint32_t>(i >> 32));
  float u1 = (static_cast<float>(a >> 8) + 1.0f) * (1.0f / 16777217.0f);
  float u2 = static_cast<float>(b >> 8) * (1.0f / 16777216.0f);
  out[i] = std_dev * sqrtf(-2.0f * logf(u1)) * cosf(6.2831853f * u2);
}

Tensor random_matrix(std::vector<int64_t> shape, uint32_t& seed) {
  Tensor t = device_tensor(std::move(shape));
  const size_t n = t.buffer.bytes / sizeof(float);
  fill_normal<<<static_cast<unsigned>((n + 255) / 256), 256>>>(static_cast<float*>(t.buffer.ptr), n,
                                                               seed, 0.02f);
  CUDA_OK(cudaGetLastError());
  seed = seed * 1664525U + 1013904223U;
  return t;
}

Tensor constant_vector(int64_t n, float v) {
  return upload(std::vector<float>(static_cast<size_t>(n), v), {n});
}

FalconH1Weights random_weights(const ModelConfig& cfg, uint32_t seed) {
  const Dims d = dims_of(cfg);
  FalconH1Weights w;
  w.embeddings = random_matrix({d.V, d.D}, seed);
  w.norm_f = constant_vector(d.D, 1.f);
  if (!cfg.tie_word_embeddings)
    w.lm_head = random_matrix({d.V, d.D}, seed);
  w.layers.resize(static_cast<size_t>(cfg.num_hidden_layers));
  uint64_t lcg = 0x2545F4914F6CDD1DULL ^ seed;
  auto uniform = [&lcg]() {
    lcg = lcg * 6364136223846793005ULL + 1442695040888963407ULL;
    return static_cast<double>(lcg >> 11) * (1.0 / 9007199254740992.0);
  };
  for (auto& L : w.layers) {
    L.ff_up_proj = random_matrix({d.F, d.D}, seed);
    L.ff_gate_proj = random_matrix({d.F, d.D}, seed);
    L.ff_down_proj = random_matrix({d.D, d.F}, seed);
    std::vector<float> a_log(static_cast<size_t>(d.H)), dt_bias(static_cast<size_t>(d.H));
    for (int64_t h = 0; h < d.H; ++h) {
      a_log[static_cast<size_t>(h)] = static_cast<float>(std::log(1.0 + 15.0 * uniform()));
      const double dt = std::exp(std::log(1e-3) + uniform() * (std::log(0.1) - std::log(1e-3)));
      dt_bias[static_cast<size_t>(h)] = static_cast<float>(dt + std::log(-std::expm1(-dt)));
    }
    L.A_log = upload(a_log, {d.H});
    L.dt_bias = upload(dt_bias, {d.H});
    L.D = constant_vector(d.H, 1.f);
    L.conv1d = random_matrix({d.conv_dim, d.K}, seed);
    L.conv1d_bias = random_matrix({d.conv_dim}, seed);
    L.in_proj = random_matrix({d.proj, d.D}, seed);
    L.out_proj = random_matrix({d.D, d.I}, seed);
    L.input_layernorm = constant_vector(d.D, 1.f);
    L.pre_ff_layer_norm = constant_vector(d.D, 1.f);
    L.q_proj = random_matrix({d.q_dim, d.D}, seed);
    L.k_proj = random_matrix({d.kv_dim, d.D}, seed);
    L.v_proj = random_matrix({d.kv_dim, d.D}, seed);
    L.o_proj = random_matrix({d.D, d.q_dim}, seed);
  }
  CUDA_OK(cudaDeviceSynchronize());
  return w;
}

// ---------------------------------------------------------------------------------------------
std::vector<int32_t> parse_ints(const std::string& s) {
  std::vector<int32_t> out;
  std::stringstream ss(s);
  std::string item;
  while (std::getline(ss, item, ','))
    if (!item.empty())
      out.push_back(static_cast<int32_t>(std::stol(item)));
  return out;
}

std::vector<float> logits_to_host(Tensor& logits) {
  std::vector<float> host(logits.buffer.bytes / sizeof(float));
  CUDA_OK(cudaMemcpy(host.data(), logits.buffer.ptr, logits.buffer.bytes, cudaMemcpyDeviceToHost));
  return host;
}

// Host argmax over logits copied from the device; first index wins ties
// (src/runtime/worker.cpp:30-59, benchmarks/generate_bench.cpp:57-94).
int32_t host_argmax(Tensor& logits, std::vector<float>& scratch) {
  const size_t n = logits.buffer.bytes / sizeof(float);
  scratch.resize(n);
  CUDA_OK(cudaMemcpy(scratch.data(), logits.buffer.ptr, n * sizeof(float), cudaMemcpyDeviceToHost));
  int32_t best = 0;
  float best_v = scratch[0];
  for (size_t i = 1; i < n; ++i)
    if (scratch[i] > best_v) {
      best_v = scratch[i];
      best = static_cast<int32_t>(i);
    }
  return best;
}

struct Args {
  std::map<std::string, std::string> kv;
  std::string get(const std::string& k, const std::string& dflt = "") const {
    auto it = kv.find(k);
    return it == kv.end() ? dflt : it->second;
  }
  long num(const std::string& k, long dflt) const {
    auto it = kv.find(k);
    return it == kv.end() ? dflt : std::stol(it->second);
  }
};

using Clock = std::chrono::steady_clock;
double seconds(Clock::time_point a, Clock::time_point b) {
  return std::chrono::duration<double>(b - a).count();
}

double percentile_ms(std::vector<double> s, double p) {  // benchmarks/generate_bench.cpp:96-107
  if (s.empty())
    return 0.0;
  std::sort(s.begin(), s.end());
  const double idx = (p / 100.0) * static_cast<double>(s.size() - 1);
  const size_t lo = static_cast<size_t>(std::floor(idx)), hi = static_cast<size_t>(std::ceil(idx));
  if (lo == hi)
    return s[lo] * 1e3;
  const double w = idx - static_cast<double>(lo);
  return (s[lo] * (1.0 - w) + s[hi] * w) * 1e3;
}

int run_logits(const Args& a) {
  const std::string dir = a.get("model");
  const int max_seq = static_cast<int>(a.num("max-seq", 256));
  const std::vector<int32_t> prompt = parse_ints(a.get("tokens"));
  const std::vector<int32_t> forced = parse_ints(a.get("decode"));
  if (prompt.empty())
    die("--tokens is empty");
  ModelConfig cfg = read_config(dir, max_seq);
  auto alloc_or = create_device_allocator(Device::GPU, 0);
  if (!alloc_or.ok())
    die(alloc_or.status().message());
  std::unique_ptr<DeviceAllocator> alloc = std::move(alloc_or.value());
  FalconH1Weights weights;
  {
    AllocatorScope scope(alloc.get());
    weights = load_weights(cfg, dir);
  }
  auto pool_or = create_cache_pool(cfg, alloc.get(), 1, create_cache_layout);
  if (!pool_or.ok())
    die(pool_or.status().message());
  std::unique_ptr<CachePool> pool = std::move(pool_or.value());
  FalconH1Runner runner(cfg, std::move(weights), cuda_ops(0));

  auto handle_or = pool->acquire();
  if (!handle_or.ok())
    die(handle_or.status().message());
  CacheHandle handle = handle_or.value();
  auto layers = pool->layer_views(handle);
  if (!layers.ok())
    die(layers.status().message());

  std::vector<float> all;
  {
    AllocatorScope scope(alloc.get());
    StatusOr<Tensor> pre = runner.prefill(ExecContext{}, prompt, layers.value());
    CUDA_OK(cudaDeviceSynchronize());
    if (!pre.ok())
      die("prefill: " + pre.status().message());
    std::vector<float> row = logits_to_host(pre.value());
    all.insert(all.end(), row.begin(), row.end());
    int64_t past = static_cast<int64_t>(prompt.size());
    for (int32_t tok : forced) {
      StatusOr<Tensor> dec = runner.decode(ExecContext{}, tok, layers.value(), past);
      CUDA_OK(cudaDeviceSynchronize());
      if (!dec.ok())
        die("decode: " + dec.status().message());
      row = logits_to_host(dec.value());
      all.insert(all.end(), row.begin(), row.end());
      ++past;
    }
  }
  std::ofstream out(a.get("out"), std::ios::binary);
  if (!out)
    die("cannot write " + a.get("out"));
  out.write(reinterpret_cast<const char*>(all.data()), static_cast<std::streamsize>(all.size() * 4));
  out.close();
  (void)pool->release(handle);
  std::printf("{\"rows\": %zu, \"vocab\": %d}\n", 1 + forced.size(), cfg.vocab_size);
  return 0;
}

struct SlotCtx {
  CacheHandle handle;
  std::span<LayerCacheView> layers;
  cudaStream_t stream = nullptr;
  cublasHandle_t cublas = nullptr;
  cudaEvent_t done = nullptr, t_start = nullptr, t_stop = nullptr;
  Tensor logits;
  int32_t cur = 1;
};

int run_bench(const Args& a) {
  const std::string dir = a.get("config");
  const int batch = static_cast<int>(a.num("batch", 1));
  const int context = static_cast<int>(a.num("context", 4096));
  const int steps = static_cast<int>(a.num("steps", 20));
  const int warmup = static_cast<int>(a.num("warmup", 3));
  const int prefill_len = static_cast<int>(a.num("prefill-len", 2048));
  const bool run_prompts = a.num("run-prompts", 1) != 0;
  const int max_seq = context + 64;
  const int prompt_len = context - steps - warmup;
  if (prompt_len < 1)
    die("context too short for the requested steps");

  ModelConfig cfg = read_config(dir, max_seq);
  auto alloc_or = create_device_allocator(Device::GPU, 0);
  if (!alloc_or.ok())
    die(alloc_or.status().message());
  std::unique_ptr<DeviceAllocator> alloc = std::move(alloc_or.value());
  FalconH1Weights weights;
  {
    AllocatorScope scope(alloc.get());
    weights = random_weights(cfg, static_cast<uint32_t>(a.num("seed", 2)));
  }
  auto pool_or = create_cache_pool(cfg, alloc.get(), batch, create_cache_layout);
  if (!pool_or.ok())
    die(pool_or.status().message());
  std::unique_ptr<CachePool> pool = std::move(pool_or.value());
  FalconH1Runner runner(cfg, std::move(weights), cuda_ops(0));

  uint64_t lcg = 0x9E3779B97F4A7C15ULL;
  auto next_token = [&]() {
    lcg = lcg * 6364136223846793005ULL + 1442695040888963407ULL;
    return static_cast<int32_t>((lcg >> 33) % static_cast<uint64_t>(cfg.vocab_size));
  };

  std::vector<SlotCtx> slots(static_cast<size_t>(batch));
  for (SlotCtx& s : slots) {
    auto h = pool->acquire();
    if (!h.ok())
      die(h.status().message());
    s.handle = h.value();
    auto lv = pool->layer_views(s.handle);
    if (!lv.ok())
      die(lv.status().message());
    s.layers = lv.value();
    if (batch > 1) {  // src/runtime/worker.cpp:121-142
      CUDA_OK(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking));
      if (cublasCreate(&s.cublas) != CUBLAS_STATUS_SUCCESS)
        die("cublasCreate failed");
      if (cublasSetStream(s.cublas, s.stream) != CUBLAS_STATUS_SUCCESS)
        die("cublasSetStream failed");
    }
    CUDA_OK(cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming));
    CUDA_OK(cudaEventCreate(&s.t_start));
    CUDA_OK(cudaEventCreate(&s.t_stop));
  }
  auto ctx_of = [&](SlotCtx& s) {
    ExecContext c;
    c.stream = s.stream;
    c.cublas = s.cublas;
    return c;
  };

  std::vector<float> scratch;
  double prompt_s = 0.0;
  // Fill the caches up to prompt_len.  With --run-prompts 0 the prompts are not run and the slots
  // keep the zeros the pool starts with: the decode kernels' time does not depend on the values.
  if (run_prompts) {
    const auto t0 = Clock::now();
    for (SlotCtx& s : slots) {
      std::vector<int32_t> prompt(static_cast<size_t>(prompt_len));
      for (auto& t : prompt)
        t = next_token();
      AllocatorScope scope(alloc.get());
      StatusOr<Tensor> pre = runner.prefill(ExecContext{}, prompt, s.layers);
      CUDA_OK(cudaDeviceSynchronize());
      if (!pre.ok())
        die("prefill: " + pre.status().message());
      s.cur = host_argmax(pre.value(), scratch);
    }
    prompt_s = seconds(t0, Clock::now());
  }

  std::vector<double> itl;
  double device_ms = 0.0, wall_s = 0.0;
  {
    AllocatorScope scope(alloc.get());
    Clock::time_point t_begin{};
    for (int step = 0; step < steps + warmup; ++step) {
      if (step == warmup) {
        CUDA_OK(cudaDeviceSynchronize());
        t_begin = Clock::now();
        for (SlotCtx& s : slots)
          CUDA_OK(cudaEventRecord(s.t_start, s.stream));
      }
      const auto t0 = Clock::now();
      const int64_t past = prompt_len + step;
      if (batch == 1) {  // benchmarks/generate_bench.cpp:329-357
        SlotCtx& s = slots[0];
        StatusOr<Tensor> dec = runner.decode(ExecContext{}, s.cur, s.layers, past);
        CUDA_OK(cudaDeviceSynchronize());
        if (!dec.ok())
          die("decode: " + dec.status().message());
        s.cur = host_argmax(dec.value(), scratch);
        CUDA_OK(cudaDeviceSynchronize());
      } else {
        for (SlotCtx& s : slots) {
          StatusOr<Tensor> dec = runner.decode(ctx_of(s), s.cur, s.layers, past);
          if (!dec.ok())
            die("decode: " + dec.status().message());
          s.logits = std::move(dec.value());
          CUDA_OK(cudaEventRecord(s.done, s.stream));
        }
        for (SlotCtx& s : slots) {
          CUDA_OK(cudaEventSynchronize(s.done));
          s.cur = host_argmax(s.logits, scratch);
          s.logits = Tensor{};
        }
      }
      if (step >= warmup)
        itl.push_back(seconds(t0, Clock::now()));
    }
    for (SlotCtx& s : slots)
      CUDA_OK(cudaEventRecord(s.t_stop, s.stream));
    CUDA_OK(cudaDeviceSynchronize());
    wall_s = seconds(t_begin, Clock::now());
    for (SlotCtx& s : slots) {
      float ms = 0.f;
      CUDA_OK(cudaEventElapsedTime(&ms, s.t_start, s.t_stop));
      device_ms = std::max(device_ms, static_cast<double>(ms));
    }
  }
  for (SlotCtx& s : slots)
    (void)pool->release(s.handle);

  // One prompt in one call, timed as BM_Prefill does: prefill + host argmax between synchronizes.
  double prefill_ms = 0.0;
  if (prefill_len > 0 && prefill_len <= max_seq) {
    std::vector<int32_t> prompt(static_cast<size_t>(prefill_len));
    for (auto& t : prompt)
      t = next_token();
    std::vector<double> times;
    for (int it = 0; it < 3; ++it) {
      auto h = pool->acquire();
      if (!h.ok())
        die(h.status().message());
      CacheHandle handle = h.value();
      auto lv = pool->layer_views(handle);
      cudaEvent_t e0, e1;
      CUDA_OK(cudaEventCreate(&e0));
      CUDA_OK(cudaEventCreate(&e1));
      CUDA_OK(cudaDeviceSynchronize());
      CUDA_OK(cudaEventRecord(e0, nullptr));
      {
        AllocatorScope scope(alloc.get());
        StatusOr<Tensor> pre = runner.prefill(ExecContext{}, prompt, lv.value());
        CUDA_OK(cudaEventRecord(e1, nullptr));
        CUDA_OK(cudaDeviceSynchronize());
        if (!pre.ok())
          die("prefill: " + pre.status().message());
        (void)host_argmax(pre.value(), scratch);
      }
      float ms = 0.f;
      CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
      if (it > 0)
        times.push_back(ms);
      CUDA_OK(cudaEventDestroy(e0));
      CUDA_OK(cudaEventDestroy(e1));
      (void)pool->release(handle);
    }
    std::sort(times.begin(), times.end());
    prefill_ms = times[times.size() / 2];
  }

  double itl_mean = 0.0;
  for (double v : itl)
    itl_mean += v;
  itl_mean = itl.empty() ? 0.0 : itl_mean / static_cast<double>(itl.size()) * 1e3;
  std::printf("{\"batch\": %d, \"steps\": %d, \"warmup\": %d, \"context\": %d, \"prompt_len\": %d, "
              "\"device_ms\": %.4f, \"wall_s\": %.6f, \"decode_tok_s_device\": %.3f, "
              "\"decode_tok_s_e2e\": %.3f, \"itl_mean_ms\": %.4f, \"itl_p50_ms\": %.4f, "
              "\"itl_p95_ms\": %.4f, \"prefill_tokens\": %d, \"prefill_ms\": %.4f, "
              "\"prompts_run\": %s, \"prompt_s\": %.3f, \"logit_bytes_d2h_per_step\": %lld}\n",
              batch, steps, warmup, context, prompt_len, device_ms, wall_s,
              batch * static_cast<double>(steps) / (device_ms / 1e3),
              batch * static_cast<double>(steps) / wall_s, itl_mean, percentile_ms(itl, 50.0),
              percentile_ms(itl, 95.0), prefill_len, prefill_ms, run_prompts ? "true" : "false",
              prompt_s, static_cast<long long>(batch) * cfg.vocab_size * 4LL);
  return 0;
}

}  // namespace

int main(int argc, char** argv) {
  if (argc < 2)
    die("usage: ref_driver logits|bench --key value ...");
  Args a;
  for (int i = 2; i + 1 < argc; i += 2) {
    std::string k = argv[i];
    if (k.rfind("--", 0) != 0)
      die("bad option " + k);
    a.kv[k.substr(2)] = argv[i + 1];
  }
  CUDA_OK(cudaSetDevice(0));
  const std::string mode = argv[1];
  if (mode == "logits")
    return run_logits(a);
  if (mode == "bench")
    return run_bench(a);
  die("unknown mode " + mode);
}
