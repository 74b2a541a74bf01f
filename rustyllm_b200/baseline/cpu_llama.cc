// A plain float32 CPU implementation of the Llama dense decoder: one token of one sequence
// against a cache, in the order of operations of SimonWaldherr/RustyLLM's `forward_into`
// (src/model.rs:7177-7358).  It is the timed CPU baseline of this library's benchmark and a
// second, independent restatement of the formulas for the tests; nothing on the GPU path
// uses it.  It is NOT RustyLLM's code and its speed is not RustyLLM's: matrix rows are dealt to
// OpenMP threads and the inner products are left to the compiler's vectoriser.
//
//   embedding row (7193) -> per layer: RMSNorm (5429-5437), q/k/v = W x (+ bias) (7207-7217),
//   rotary encoding of q and k (half-split pairs 5606-5647, or interleaved pairs 5562-5603),
//   K[pos] = k, V[pos] = v (7233-7236), per head a streaming softmax over positions 0..pos
//   (5807-5869) with scale 1/sqrt(head_dim), x += Wo attn (7315-7318), RMSNorm,
//   x += Wdown (silu(Wgate xn) * (Wup xn)) (7321-7347; silu as in src/simd.rs:2403-2408)
//   -> RMSNorm -> logits = Wout xn (7351-7357).
//
// All tensors are float32 and borrowed from the caller, who keeps them alive.  Layer l uses
// the weights set for layer (l mod layers_set): a timing run of a deep model may thus hold
// fewer distinct layers than it runs (each pass still streams a layer's weights from memory).
#include <math.h>
#include <stdint.h>
#include <string.h>

#include <vector>

#ifdef _OPENMP
#include <omp.h>
#endif

namespace {

struct LayerWeights {
  const float *attn_norm, *wq, *wk, *wv, *bq, *bk, *bv, *wo, *ffn_norm, *w_gate, *w_up, *w_down;
};

struct CpuLlama {
  int dim, n_layers, n_heads, n_kv_heads, head_dim, hidden, vocab, max_seq, interleaved;
  float eps;
  std::vector<float> inv_freq;
  std::vector<LayerWeights> layers;       // distinct layers held; layer l runs layers[l % size]
  const float *embed = nullptr, *out_norm = nullptr, *out = nullptr;
  std::vector<float> x, xn, q, k, v, attn, proj, gate, up, hid;
  std::vector<std::vector<float>> k_cache, v_cache;   // per layer: [max_seq, n_kv_heads * head_dim]
};

inline float dot(const float* a, const float* b, int n) {
  float s = 0.0f;
#pragma omp simd reduction(+ : s)
  for (int i = 0; i < n; ++i) s += a[i] * b[i];
  return s;
}

// y = W x (+ bias): W is [rows, cols] row-major, `out = W . x` as src/model.rs:185-186
void matvec(const float* w, const float* x, const float* bias, float* y, int rows, int cols) {
#pragma omp parallel for schedule(static)
  for (int r = 0; r < rows; ++r) {
    const float s = dot(w + (size_t)r * cols, x, cols);
    y[r] = bias ? s + bias[r] : s;
  }
}

void rms_norm(const float* x, const float* w, float eps, float* out, int n) {
  const float ss = dot(x, x, n) / (float)n;
  const float scale = 1.0f / sqrtf(ss + eps);
  for (int i = 0; i < n; ++i) out[i] = x[i] * scale * w[i];
}

void rope(float* vec, int heads, int head_dim, int pos, const float* inv_freq, int interleaved) {
  const int half = head_dim / 2;
  for (int i = 0; i < half; ++i) {
    const float angle = (float)pos * inv_freq[i];
    const float s = sinf(angle), c = cosf(angle);
    for (int h = 0; h < heads; ++h) {
      float* p = vec + (size_t)h * head_dim;
      const int i0 = interleaved ? 2 * i : i, i1 = interleaved ? 2 * i + 1 : i + half;
      const float v0 = p[i0], v1 = p[i1];
      p[i0] = v0 * c - v1 * s;
      p[i1] = v0 * s + v1 * c;
    }
  }
}

// one query head over positions 0..pos of one KV head: running maximum, denominator and
// output, rescaled when a larger score arrives
void attend(const float* q, const float* keys, const float* values, int stride, int head_dim, int pos, float scale,
            float* out) {
  float max_score = -INFINITY, denom = 0.0f;
  for (int i = 0; i < head_dim; ++i) out[i] = 0.0f;
  for (int t = 0; t <= pos; ++t) {
    const float score = dot(q, keys + (size_t)t * stride, head_dim) * scale;
    const float* vrow = values + (size_t)t * stride;
    if (score > max_score) {
      const float old = isfinite(max_score) ? expf(max_score - score) : 0.0f;
      for (int i = 0; i < head_dim; ++i) out[i] = out[i] * old + vrow[i];
      denom = denom * old + 1.0f;
      max_score = score;
    } else {
      const float w = expf(score - max_score);
      for (int i = 0; i < head_dim; ++i) out[i] += w * vrow[i];
      denom += w;
    }
  }
  if (denom > 0.0f) {
    const float inv = 1.0f / denom;
    for (int i = 0; i < head_dim; ++i) out[i] *= inv;
  }
}

}  // namespace

extern "C" {

// dims: dim, layers, heads, kv_heads, head_dim, hidden (feed-forward width), vocab, max_seq
void* cpu_llama_new(const int* dims, float eps, const float* inv_freq, int rope_interleaved) {
  for (int i = 0; i < 8; ++i)
    if (dims[i] <= 0) return nullptr;
  if (dims[2] % dims[3] != 0 || dims[4] % 2 != 0) return nullptr;
  CpuLlama* m = new CpuLlama();
  m->dim = dims[0]; m->n_layers = dims[1]; m->n_heads = dims[2]; m->n_kv_heads = dims[3];
  m->head_dim = dims[4]; m->hidden = dims[5]; m->vocab = dims[6]; m->max_seq = dims[7];
  m->eps = eps; m->interleaved = rope_interleaved;
  m->inv_freq.assign(inv_freq, inv_freq + m->head_dim / 2);
  const int qd = m->n_heads * m->head_dim, kvd = m->n_kv_heads * m->head_dim;
  m->x.resize(m->dim); m->xn.resize(m->dim); m->proj.resize(m->dim);
  m->q.resize(qd); m->attn.resize(qd); m->k.resize(kvd); m->v.resize(kvd);
  m->gate.resize(m->hidden); m->up.resize(m->hidden); m->hid.resize(m->hidden);
  m->k_cache.assign(m->n_layers, std::vector<float>((size_t)m->max_seq * kvd));
  m->v_cache.assign(m->n_layers, std::vector<float>((size_t)m->max_seq * kvd));
  return m;
}

void cpu_llama_free(void* h) { delete (CpuLlama*)h; }

// ptrs: attn_norm, wq, wk, wv, bq, bk, bv (the three biases may be null), wo, ffn_norm, gate, up, down.
// Layers are set in order 0, 1, ...; at most as many as the model runs.
int cpu_llama_add_layer(void* h, const float* const* ptrs) {
  CpuLlama* m = (CpuLlama*)h;
  if ((int)m->layers.size() >= m->n_layers) return -1;
  LayerWeights w = {ptrs[0], ptrs[1], ptrs[2], ptrs[3], ptrs[4], ptrs[5], ptrs[6], ptrs[7], ptrs[8], ptrs[9], ptrs[10], ptrs[11]};
  if (!w.attn_norm || !w.wq || !w.wk || !w.wv || !w.wo || !w.ffn_norm || !w.w_gate || !w.w_up || !w.w_down) return -1;
  m->layers.push_back(w);
  return 0;
}

int cpu_llama_set_globals(void* h, const float* embed, const float* out_norm, const float* out) {
  CpuLlama* m = (CpuLlama*)h;
  if (!embed || !out_norm || !out) return -1;
  m->embed = embed; m->out_norm = out_norm; m->out = out;
  return 0;
}

int cpu_llama_threads() {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

// One token at position pos (positions must come in order 0, 1, 2, ... for a sequence; a new
// sequence simply starts again at 0).  logits: [vocab], or null to skip the head (a prompt
// token whose logits nobody reads, as src/model.rs:9801 does).
int cpu_llama_forward(void* h, int token, int pos, float* logits) {
  CpuLlama* m = (CpuLlama*)h;
  if (!m || m->layers.empty() || !m->embed) return -1;
  if (token < 0 || token >= m->vocab || pos < 0 || pos >= m->max_seq) return -2;
  const int dim = m->dim, hd = m->head_dim, H = m->n_heads, G = m->n_kv_heads;
  const int qd = H * hd, kvd = G * hd, kv_mul = H / G;
  const float scale = 1.0f / sqrtf((float)hd);
  memcpy(m->x.data(), m->embed + (size_t)token * dim, sizeof(float) * dim);
  for (int l = 0; l < m->n_layers; ++l) {
    const LayerWeights& w = m->layers[l % m->layers.size()];
    rms_norm(m->x.data(), w.attn_norm, m->eps, m->xn.data(), dim);
    matvec(w.wq, m->xn.data(), w.bq, m->q.data(), qd, dim);
    matvec(w.wk, m->xn.data(), w.bk, m->k.data(), kvd, dim);
    matvec(w.wv, m->xn.data(), w.bv, m->v.data(), kvd, dim);
    rope(m->q.data(), H, hd, pos, m->inv_freq.data(), m->interleaved);
    rope(m->k.data(), G, hd, pos, m->inv_freq.data(), m->interleaved);
    float* kc = m->k_cache[l].data();
    float* vc = m->v_cache[l].data();
    memcpy(kc + (size_t)pos * kvd, m->k.data(), sizeof(float) * kvd);
    memcpy(vc + (size_t)pos * kvd, m->v.data(), sizeof(float) * kvd);
#pragma omp parallel for schedule(static)
    for (int hh = 0; hh < H; ++hh) {
      const int g = hh / kv_mul;       // contiguous groups of query heads share a KV head
      attend(m->q.data() + (size_t)hh * hd, kc + (size_t)g * hd, vc + (size_t)g * hd, kvd, hd, pos, scale,
             m->attn.data() + (size_t)hh * hd);
    }
    matvec(w.wo, m->attn.data(), nullptr, m->proj.data(), dim, qd);
    for (int i = 0; i < dim; ++i) m->x[i] += m->proj[i];
    rms_norm(m->x.data(), w.ffn_norm, m->eps, m->xn.data(), dim);
    matvec(w.w_gate, m->xn.data(), nullptr, m->gate.data(), m->hidden, dim);
    matvec(w.w_up, m->xn.data(), nullptr, m->up.data(), m->hidden, dim);
    for (int i = 0; i < m->hidden; ++i) {
      const float g = m->gate[i];
      m->hid[i] = g / (1.0f + expf(-g)) * m->up[i];
    }
    matvec(w.w_down, m->hid.data(), nullptr, m->proj.data(), dim, m->hidden);
    for (int i = 0; i < dim; ++i) m->x[i] += m->proj[i];
  }
  if (logits) {
    rms_norm(m->x.data(), m->out_norm, m->eps, m->xn.data(), dim);
    matvec(m->out, m->xn.data(), nullptr, logits, m->vocab, dim);
  }
  return 0;
}

}  // extern "C"
