// A second, independent writing of the dense Qwen3 forward pass, for tests only.
//
// tests/plain_qwen3.py restates the reference's CPU path
// (crates/model/src/qwen35/cpu.rs) as whole-sequence tensor expressions.  This
// file restates the reference's OTHER writing of the same model, the teaching
// engine of crates/lab/src/engine.rs:275-406, in its own manner: scalar loops,
// in-place operations, a key/value cache that a prompt step and then
// single-token steps append to, and a dot product with eight running sums
// (engine.rs:455-465).  The two share no code and not even a language; where
// they agree to float32 rounding, both read the formulas the same way.  The
// reference itself (Rust over GGUF) cannot be compiled where these tests run,
// so neither writing is checked against its output.
//
// It reads the model folder by itself (config.json and model.safetensors, with
// a small JSON reader of its own) and shares nothing with llmoxide_b200.
//
//   qwen3_twin MODEL_DIR OUT_FILE PREFIX_LEN tok0 tok1 ...
// feeds the first PREFIX_LEN tokens as one step and the others one by one, and
// writes the logits of every position as little-endian float32 [T, vocab].
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <string>
#include <vector>

// ---------------------------------------------------------------------------
// A JSON reader, as small as the two files need.
// ---------------------------------------------------------------------------
struct Json {
  enum Kind { Null, Bool, Num, Str, Arr, Obj } kind = Null;
  bool b = false;
  double num = 0;
  std::string str;
  std::vector<Json> arr;
  std::vector<std::pair<std::string, Json>> obj;
  const Json* get(const std::string& key) const {
    for (auto& kv : obj)
      if (kv.first == key) return &kv.second;
    return nullptr;
  }
};

struct JsonReader {
  const std::string& s;
  size_t at = 0;
  explicit JsonReader(const std::string& text) : s(text) {}
  [[noreturn]] void fail(const char* what) {
    std::fprintf(stderr, "json: %s at byte %zu\n", what, at);
    std::exit(2);
  }
  void skip() {
    while (at < s.size() && (s[at] == ' ' || s[at] == '\n' || s[at] == '\t' || s[at] == '\r')) ++at;
  }
  std::string string() {
    std::string out;
    ++at;  // the opening quote
    while (at < s.size() && s[at] != '"') {
      if (s[at] == '\\') {
        ++at;
        if (at >= s.size()) fail("string ends in an escape");
        const char c = s[at];
        if (c == 'n') out += '\n';
        else if (c == 't') out += '\t';
        else if (c == 'u') { out += '?'; at += 4; }
        else out += c;
      } else {
        out += s[at];
      }
      ++at;
    }
    if (at >= s.size()) fail("string without an end");
    ++at;
    return out;
  }
  Json value() {
    skip();
    if (at >= s.size()) fail("value expected");
    Json j;
    const char c = s[at];
    if (c == '{') {
      j.kind = Json::Obj;
      ++at;
      skip();
      if (s[at] == '}') { ++at; return j; }
      for (;;) {
        skip();
        if (s[at] != '"') fail("key expected");
        std::string key = string();
        skip();
        if (s[at] != ':') fail("colon expected");
        ++at;
        Json v = value();
        j.obj.emplace_back(std::move(key), std::move(v));
        skip();
        if (s[at] == ',') { ++at; continue; }
        if (s[at] == '}') { ++at; return j; }
        fail("comma or brace expected");
      }
    }
    if (c == '[') {
      j.kind = Json::Arr;
      ++at;
      skip();
      if (s[at] == ']') { ++at; return j; }
      for (;;) {
        j.arr.push_back(value());
        skip();
        if (s[at] == ',') { ++at; continue; }
        if (s[at] == ']') { ++at; return j; }
        fail("comma or bracket expected");
      }
    }
    if (c == '"') {
      j.kind = Json::Str;
      j.str = string();
      return j;
    }
    if (!s.compare(at, 4, "true")) { j.kind = Json::Bool; j.b = true; at += 4; return j; }
    if (!s.compare(at, 5, "false")) { j.kind = Json::Bool; at += 5; return j; }
    if (!s.compare(at, 4, "null")) { at += 4; return j; }
    char* end = nullptr;
    j.num = std::strtod(s.c_str() + at, &end);
    if (end == s.c_str() + at) fail("number expected");
    j.kind = Json::Num;
    at = (size_t)(end - s.c_str());
    return j;
  }
};

static std::string read_file(const std::string& path) {
  std::ifstream f(path, std::ios::binary);
  if (!f) {
    std::fprintf(stderr, "cannot open %s\n", path.c_str());
    std::exit(2);
  }
  std::ostringstream ss;
  ss << f.rdbuf();
  return ss.str();
}

// ---------------------------------------------------------------------------
// The model folder
// ---------------------------------------------------------------------------
struct Tensor {
  std::vector<int64_t> shape;
  std::vector<float> data;
};

static float bf16_to_f32(uint16_t h) {
  uint32_t u = (uint32_t)h << 16;
  float f;
  std::memcpy(&f, &u, 4);
  return f;
}

// safetensors: u64 header length, JSON header {name: {dtype, shape, data_offsets}}, payload
static std::map<std::string, Tensor> read_safetensors(const std::string& path) {
  const std::string raw = read_file(path);
  uint64_t n = 0;
  std::memcpy(&n, raw.data(), 8);
  const std::string header = raw.substr(8, n);
  JsonReader rd(header);
  const Json h = rd.value();
  const char* payload = raw.data() + 8 + n;
  std::map<std::string, Tensor> out;
  for (auto& kv : h.obj) {
    if (kv.first == "__metadata__") continue;
    const Json& info = kv.second;
    Tensor t;
    size_t count = 1;
    for (auto& d : info.get("shape")->arr) {
      t.shape.push_back((int64_t)d.num);
      count *= (size_t)d.num;
    }
    const size_t lo = (size_t)info.get("data_offsets")->arr[0].num;
    const std::string& dt = info.get("dtype")->str;
    t.data.resize(count);
    if (dt == "F32") {
      std::memcpy(t.data.data(), payload + lo, count * 4);
    } else if (dt == "BF16") {
      for (size_t i = 0; i < count; ++i) {
        uint16_t v;
        std::memcpy(&v, payload + lo + 2 * i, 2);
        t.data[i] = bf16_to_f32(v);
      }
    } else {
      std::fprintf(stderr, "%s: dtype %s is not read by the twin\n", kv.first.c_str(), dt.c_str());
      std::exit(2);
    }
    out.emplace(kv.first, std::move(t));
  }
  return out;
}

struct Config {
  int n_layers, d_model, ffn_dim, n_heads, n_kv_heads, head_dim, vocab;
  float rms_eps, rope_base;
  std::vector<int> window;   // per layer, 0 = every earlier key
};

static double num_or(const Json& j, const char* key, double fallback) {
  const Json* v = j.get(key);
  return (v && v->kind == Json::Num) ? v->num : fallback;
}

static Config read_config(const std::string& path) {
  const std::string text = read_file(path);
  JsonReader rd(text);
  const Json j = rd.value();
  Config c;
  c.n_layers = (int)num_or(j, "num_hidden_layers", 0);
  c.d_model = (int)num_or(j, "hidden_size", 0);
  c.ffn_dim = (int)num_or(j, "intermediate_size", 0);
  c.n_heads = (int)num_or(j, "num_attention_heads", 0);
  c.n_kv_heads = (int)num_or(j, "num_key_value_heads", c.n_heads);        // engine.rs:88
  c.head_dim = (int)num_or(j, "head_dim", c.n_heads ? c.d_model / c.n_heads : 0);   // engine.rs:70
  c.vocab = (int)num_or(j, "vocab_size", 0);
  c.rms_eps = (float)num_or(j, "rms_norm_eps", 0);
  c.rope_base = (float)num_or(j, "rope_theta", 10000.0);                    // engine.rs:92
  // Which layers look through a window: config.json's layer_types, else use_sliding_window with
  // max_window_layers.  The lab engine has no window; the visible range is crates/model/src/cache.rs:31-37.
  c.window.assign(c.n_layers, 0);
  const int w = (int)num_or(j, "sliding_window", 0);
  const Json* types = j.get("layer_types");
  const Json* use = j.get("use_sliding_window");
  if (types && types->kind == Json::Arr) {
    for (int i = 0; i < c.n_layers && i < (int)types->arr.size(); ++i)
      if (types->arr[i].str == "sliding_attention") c.window[i] = w;
  } else if (use && use->kind == Json::Bool && use->b && w > 0) {
    const int first = (int)num_or(j, "max_window_layers", c.n_layers);
    for (int i = first; i < c.n_layers; ++i) c.window[i] = w;
  }
  return c;
}

// ---------------------------------------------------------------------------
// Operations (crates/model/src/ops.rs and crates/lab/src/engine.rs)
// ---------------------------------------------------------------------------

// engine.rs:455-465: eight running sums, then their sum, then the tail
static float dot(const float* a, const float* b, int n) {
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  const int whole = n / 8 * 8;
  float tail = 0.f;
  for (int i = whole; i < n; ++i) tail += a[i] * b[i];
  for (int i = 0; i < whole; i += 8)
    for (int j = 0; j < 8; ++j) acc[j] += a[i + j] * b[i + j];
  float s = 0.f;
  for (int j = 0; j < 8; ++j) s += acc[j];
  return s + tail;
}

// engine.rs:435-447: y[i, o] = W[o, :] . x[i, :]
static void matmul(float* y, const Tensor& w, const float* x, int t) {
  const int n_out = (int)w.shape[0], n_in = (int)w.shape[1];
  for (int o = 0; o < n_out; ++o)
    for (int i = 0; i < t; ++i) y[(size_t)i * n_out + o] = dot(w.data.data() + (size_t)o * n_in, x + (size_t)i * n_in, n_in);
}

// ops.rs:40-59: mean of squares in float32, one multiply by the scale, one by the gain
static void rms_norm_mul(float* x, const float* w, int n, float eps) {
  float sum = 0.f;
  for (int i = 0; i < n; ++i) sum += x[i] * x[i];
  const float mean_sq = sum / (float)n;
  const float scale = 1.0f / std::sqrt(mean_sq + eps);
  for (int i = 0; i < n; ++i) x[i] *= scale;
  for (int i = 0; i < n; ++i) x[i] *= w[i];
}

// engine.rs:470-486 (Rope::Halves): the angle is a float64 recurrence, sin and cos are rounded to float32
static void rope_halves(float* head, int d, int pos, float base) {
  const int half = d / 2;
  const double theta_scale = std::pow((double)base, -2.0 / (double)d);
  double theta = (double)pos;
  for (int i = 0; i < half; ++i) {
    const float sn = (float)std::sin(theta), cs = (float)std::cos(theta);
    const float x0 = head[i], x1 = head[i + half];
    head[i] = x0 * cs - x1 * sn;
    head[i + half] = x0 * sn + x1 * cs;
    theta *= theta_scale;
  }
}

// ops.rs:119-135
static void softmax(float* x, int n) {
  float mx = -INFINITY;
  for (int i = 0; i < n; ++i) mx = std::fmax(mx, x[i]);
  if (!std::isfinite(mx)) {
    for (int i = 0; i < n; ++i) x[i] = 0.f;
    return;
  }
  float sum = 0.f;
  for (int i = 0; i < n; ++i) {
    x[i] = std::exp(x[i] - mx);
    sum += x[i];
  }
  const float inv = 1.0f / sum;
  for (int i = 0; i < n; ++i) x[i] *= inv;
}

// ops.rs:176-178
static float silu(float x) { return x / (1.0f + std::exp(-x)); }

// ---------------------------------------------------------------------------
// The model with its cache (engine.rs:275-406)
// ---------------------------------------------------------------------------
struct Model {
  Config cfg;
  std::map<std::string, Tensor> w;
  std::vector<std::vector<float>> cache_k, cache_v;   // per layer: [position][kv_dim]
  int len = 0;

  const Tensor& tensor(const std::string& name) const {
    auto it = w.find(name);
    if (it == w.end()) {
      std::fprintf(stderr, "missing tensor %s\n", name.c_str());
      std::exit(2);
    }
    return it->second;
  }
  const Tensor& layer(int il, const char* what) const {
    return tensor("model.layers." + std::to_string(il) + "." + what);
  }

  // Appends `tokens` at position `len`; logits of every new position into out [t, vocab].
  void forward(const std::vector<int>& tokens, float* out) {
    const Config& c = cfg;
    const int t = (int)tokens.size(), d = c.d_model, hd = c.head_dim;
    const int q_dim = c.n_heads * hd, kv_dim = c.n_kv_heads * hd, base = len;
    std::vector<float> h((size_t)t * d), x((size_t)t * d), q((size_t)t * q_dim), k((size_t)t * kv_dim),
        v((size_t)t * kv_dim), attn((size_t)t * q_dim), proj((size_t)t * d), gate((size_t)t * c.ffn_dim),
        up((size_t)t * c.ffn_dim), scores;
    const Tensor& embed = tensor("model.embed_tokens.weight");
    for (int i = 0; i < t; ++i)     // one row of the table per token, no arithmetic
      std::memcpy(&h[(size_t)i * d], &embed.data[(size_t)tokens[i] * d], (size_t)d * 4);
    const int group = c.n_heads / c.n_kv_heads;
    const float scale = 1.0f / std::sqrt((float)hd);
    for (int il = 0; il < c.n_layers; ++il) {
      // --- attention ---
      x = h;
      for (int i = 0; i < t; ++i) rms_norm_mul(&x[(size_t)i * d], layer(il, "input_layernorm.weight").data.data(), d, c.rms_eps);
      matmul(q.data(), layer(il, "self_attn.q_proj.weight"), x.data(), t);
      matmul(k.data(), layer(il, "self_attn.k_proj.weight"), x.data(), t);
      matmul(v.data(), layer(il, "self_attn.v_proj.weight"), x.data(), t);
      const float* qn = layer(il, "self_attn.q_norm.weight").data.data();
      const float* kn = layer(il, "self_attn.k_norm.weight").data.data();
      for (int i = 0; i < t * c.n_heads; ++i) {
        rms_norm_mul(&q[(size_t)i * hd], qn, hd, c.rms_eps);
        rope_halves(&q[(size_t)i * hd], hd, base + i / c.n_heads, c.rope_base);
      }
      for (int i = 0; i < t * c.n_kv_heads; ++i) {
        rms_norm_mul(&k[(size_t)i * hd], kn, hd, c.rms_eps);
        rope_halves(&k[(size_t)i * hd], hd, base + i / c.n_kv_heads, c.rope_base);
      }
      // the step's keys and values join the cache, then every query attends over what it may see
      cache_k[il].insert(cache_k[il].end(), k.begin(), k.end());
      cache_v[il].insert(cache_v[il].end(), v.begin(), v.end());
      const float* layer_k = cache_k[il].data();
      const float* layer_v = cache_v[il].data();
      for (int i = 0; i < t; ++i) {
        const int pos = base + i;
        const int first = (c.window[il] > 0 && pos - (c.window[il] - 1) > 0) ? pos - (c.window[il] - 1) : 0;
        const int seen = pos + 1 - first;
        scores.resize(seen);
        for (int hq = 0; hq < c.n_heads; ++hq) {
          const int kvh = hq / group;
          const float* qv = &q[(size_t)i * q_dim + (size_t)hq * hd];
          for (int p = 0; p < seen; ++p)
            scores[p] = dot(qv, layer_k + (size_t)(first + p) * kv_dim + (size_t)kvh * hd, hd) * scale;
          softmax(scores.data(), seen);
          float* o = &attn[(size_t)i * q_dim + (size_t)hq * hd];
          for (int e = 0; e < hd; ++e) o[e] = 0.f;
          for (int p = 0; p < seen; ++p) {
            const float a = scores[p];
            const float* vv = layer_v + (size_t)(first + p) * kv_dim + (size_t)kvh * hd;
            for (int e = 0; e < hd; ++e) o[e] += a * vv[e];
          }
        }
      }
      matmul(proj.data(), layer(il, "self_attn.o_proj.weight"), attn.data(), t);
      for (size_t i = 0; i < h.size(); ++i) h[i] += proj[i];
      // --- feed-forward ---
      x = h;
      for (int i = 0; i < t; ++i)
        rms_norm_mul(&x[(size_t)i * d], layer(il, "post_attention_layernorm.weight").data.data(), d, c.rms_eps);
      matmul(gate.data(), layer(il, "mlp.gate_proj.weight"), x.data(), t);
      matmul(up.data(), layer(il, "mlp.up_proj.weight"), x.data(), t);
      for (size_t i = 0; i < gate.size(); ++i) gate[i] = silu(gate[i]) * up[i];
      matmul(proj.data(), layer(il, "mlp.down_proj.weight"), gate.data(), t);
      for (size_t i = 0; i < h.size(); ++i) h[i] += proj[i];
    }
    len = base + t;
    // the head: lm_head, or the embedding table when the folder has none (crates/model/src/qwen35/weights.rs:79)
    auto it = w.find("lm_head.weight");
    const Tensor& head = it != w.end() ? it->second : embed;
    for (int i = 0; i < t; ++i) {
      rms_norm_mul(&h[(size_t)i * d], tensor("model.norm.weight").data.data(), d, c.rms_eps);
      matmul(out + (size_t)i * c.vocab, head, &h[(size_t)i * d], 1);
    }
  }
};

int main(int argc, char** argv) {
  if (argc < 5) {
    std::fprintf(stderr, "usage: qwen3_twin MODEL_DIR OUT_FILE PREFIX_LEN tok0 tok1 ...\n");
    return 2;
  }
  const std::string dir = argv[1];
  Model m;
  m.cfg = read_config(dir + "/config.json");
  m.w = read_safetensors(dir + "/model.safetensors");
  m.cache_k.resize(m.cfg.n_layers);
  m.cache_v.resize(m.cfg.n_layers);
  const int prefix = std::atoi(argv[3]);
  std::vector<int> toks;
  for (int i = 4; i < argc; ++i) toks.push_back(std::atoi(argv[i]));
  const int T = (int)toks.size();
  if (prefix < 1 || prefix > T) {
    std::fprintf(stderr, "PREFIX_LEN must be between 1 and the number of tokens\n");
    return 2;
  }
  std::vector<float> logits((size_t)T * m.cfg.vocab);
  m.forward(std::vector<int>(toks.begin(), toks.begin() + prefix), logits.data());
  for (int i = prefix; i < T; ++i) m.forward({toks[i]}, logits.data() + (size_t)i * m.cfg.vocab);
  std::FILE* f = std::fopen(argv[2], "wb");
  if (!f) return 2;
  std::fwrite(logits.data(), 4, logits.size(), f);
  std::fclose(f);
  return 0;
}
