// Native executor of a planned inference graph on the host.
//
// The Python side (oslo_b200/lightseq/lsflow.py) declares a model's operators once, plans one arena for every
// intermediate tensor and then, for graphs made of the operators below, hands this file a flat program: one record of
// 16 int64 per operator plus a table of base pointers.  A request is then ONE call: the interpreter walks the records and
// runs each operator on the arena with the request's row count, sequence length, decoding step and padding mask.  No
// allocation happens here; the only scratch (attention scores) is a per-thread buffer sized from the program.
//
// Reference counterpart: the C++ graph runtime that executes its inference models node by node over a planned buffer
// (oslo/lightseq2/csrc/lsflow/{context,node,layer}.cpp) with the x86 kernels of oslo/lightseq2/csrc/kernels/x86.
// Everything is fp32, row-major.  Rows are tokens (batch x seq) unless a record says "one row per sequence".
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

extern "C" int oslo_cpu_sgemm(int transpose_a, int transpose_b, long long m, long long n, long long k, float alpha, const float* a,
                              long long lda, const float* b, long long ldb, float beta, float* c, long long ldc);

namespace {

enum Op : int64_t {
  kLinear = 1,           // out[rows, d1] = act(in0[rows, d0] W[d1, d0]^T + bias)
  kLayerNorm = 2,        // out[rows, d0] = LN(in0) * w + bias
  kAdd = 3,              // out = in0 + in1, [rows, d0]
  kAttention = 4,        // in0 = qkv [b, s, 3, heads=d1, hd=d2] -> out [b, s, d1 * d2]; flags bit0 = causal; padding mask
  kEmbedding = 5,        // in0 = ids (int64) -> out[rows, d0] = table[id] * scale + pos[step + t]; id == d2 -> zeros
  kSelect = 6,           // in0 [b, s, d0] -> out [b, d0], token d2 (0 = first, -1 = last)
  kActivation = 7,       // out = f(in0), f = d2: 0 tanh, 1 relu, 2 gelu(tanh)
  kCachedAttention = 8,  // like kAttention, keys / values appended to caches [max_b, heads, max_len, hd] at `step`
};

constexpr int kRecord = 16;
enum Field { fOp = 0, fIn0, fIn1, fOut, fW, fB, fRowsKind, fD0, fD1, fD2, fFlags, fScalar, fX0, fX1, fMaxLen, fReserved };

inline float as_float(int64_t bits) {
  double d;
  std::memcpy(&d, &bits, sizeof(d));
  return static_cast<float>(d);
}

inline float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;
  return 0.5f * x * (1.f + std::tanh(k * (x + 0.044715f * x * x * x)));
}

inline void apply_act(float* x, long long n, int kind) {
  if (kind == 0) for (long long i = 0; i < n; ++i) x[i] = std::tanh(x[i]);
  else if (kind == 1) for (long long i = 0; i < n; ++i) x[i] = x[i] > 0.f ? x[i] : 0.f;
  else if (kind == 2) for (long long i = 0; i < n; ++i) x[i] = gelu_tanh(x[i]);
}

void linear(const float* x, const float* w, const float* bias, float* out, long long rows, long long k, long long n, int act) {
  oslo_cpu_sgemm(0, 1, rows, n, k, 1.f, x, k, w, k, 0.f, out, n);
  if (!bias && act < 0) return;
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < rows; ++r) {
    float* o = out + r * n;
    if (bias) for (long long j = 0; j < n; ++j) o[j] += bias[j];
    if (act >= 0) apply_act(o, n, act);
  }
}

void layer_norm(const float* x, const float* w, const float* b, float* out, long long rows, long long h, float eps) {
#pragma omp parallel for schedule(static)
  for (long long r = 0; r < rows; ++r) {
    const float* xi = x + r * h;
    float* o = out + r * h;
    double mean = 0.0, var = 0.0;
    for (long long j = 0; j < h; ++j) mean += xi[j];
    mean /= static_cast<double>(h);
    for (long long j = 0; j < h; ++j) {
      const double d = xi[j] - mean;
      var += d * d;
    }
    const float inv = 1.f / std::sqrt(static_cast<float>(var / static_cast<double>(h)) + eps);
    const float m = static_cast<float>(mean);
    for (long long j = 0; j < h; ++j) o[j] = (xi[j] - m) * inv * (w ? w[j] : 1.f) + (b ? b[j] : 0.f);
  }
}

// One (batch, head) pair: q rows [s_q] against keys / values [s_k]; query i sees key j when j <= q_pos0 + i (causal) and
// the key is not padding.  q / k / v are addressed by (pointer, row stride); the result goes to out with its own stride.
void attend(const float* q, long long q_stride, const float* k, long long k_stride, const float* v, long long v_stride,
            float* out, long long out_stride, long long s_q, long long s_k, long long hd, bool causal, long long q_pos0,
            const uint8_t* key_pad, float* scores) {
  const float scale = 1.f / std::sqrt(static_cast<float>(hd));
  for (long long i = 0; i < s_q; ++i) {
    const float* qi = q + i * q_stride;
    const long long limit = causal ? std::min(s_k, q_pos0 + i + 1) : s_k;
    float mx = -INFINITY;
    for (long long j = 0; j < limit; ++j) {
      const float* kj = k + j * k_stride;
      float dot = 0.f;
      for (long long d = 0; d < hd; ++d) dot += qi[d] * kj[d];
      dot *= scale;
      if (key_pad && key_pad[j]) dot += -1e4f;  // the additive mask value of the eager path
      scores[j] = dot;
      mx = std::max(mx, dot);
    }
    float sum = 0.f;
    for (long long j = 0; j < limit; ++j) {
      scores[j] = std::exp(scores[j] - mx);
      sum += scores[j];
    }
    const float inv = sum > 0.f ? 1.f / sum : 0.f;
    float* oi = out + i * out_stride;
    for (long long d = 0; d < hd; ++d) oi[d] = 0.f;
    for (long long j = 0; j < limit; ++j) {
      const float p = scores[j] * inv;
      const float* vj = v + j * v_stride;
      for (long long d = 0; d < hd; ++d) oi[d] += p * vj[d];
    }
  }
}

}  // namespace

// prog: n_ops records of 16 int64 (see Field); ptrs: base pointers, records refer to them by index (-1 = absent).
// lead = batch * seq rows; step = position of the first token (decoding); pad = [batch, seq] bytes, nonzero at padding, or
// null.  Returns 0, or -(index + 1) of the first record it could not run.
extern "C" int oslo_cpu_graph_run(const int64_t* prog, int n_ops, void* const* ptrs, long long lead, long long seq, long long step,
                                  const uint8_t* pad) {
  if (!prog || !ptrs || seq <= 0 || lead <= 0 || lead % seq) return -1000000;
  const long long batch = lead / seq;
  long long max_keys = seq;
  for (int i = 0; i < n_ops; ++i)
    if (prog[i * kRecord + fOp] == kCachedAttention) max_keys = std::max<long long>(max_keys, prog[i * kRecord + fMaxLen]);
  for (int i = 0; i < n_ops; ++i) {
    const int64_t* r = prog + static_cast<long long>(i) * kRecord;
    auto P = [&](int f) -> void* { return r[f] < 0 ? nullptr : ptrs[r[f]]; };
    const long long rows = r[fRowsKind] == 1 ? batch : lead;
    const float* in0 = static_cast<const float*>(P(fIn0));
    float* out = static_cast<float*>(P(fOut));
    if (!out || !P(fIn0)) return -(i + 1);
    switch (r[fOp]) {
      case kLinear:
        linear(in0, static_cast<const float*>(P(fW)), static_cast<const float*>(P(fB)), out, rows, r[fD0], r[fD1],
               static_cast<int>(r[fD2]));
        break;
      case kLayerNorm:
        layer_norm(in0, static_cast<const float*>(P(fW)), static_cast<const float*>(P(fB)), out, rows, r[fD0], as_float(r[fScalar]));
        break;
      case kAdd: {
        const float* in1 = static_cast<const float*>(P(fIn1));
        if (!in1) return -(i + 1);
        const long long n = rows * r[fD0];
#pragma omp parallel for schedule(static)
        for (long long j = 0; j < n; ++j) out[j] = in0[j] + in1[j];
        break;
      }
      case kActivation: {
        const long long n = rows * r[fD0];
        if (out != in0) std::memcpy(out, in0, sizeof(float) * n);
        apply_act(out, n, static_cast<int>(r[fD2]));
        break;
      }
      case kSelect: {
        const long long h = r[fD0];
        const long long t = r[fD2] < 0 ? seq + r[fD2] : r[fD2];
        for (long long b = 0; b < batch; ++b) std::memcpy(out + b * h, in0 + (b * seq + t) * h, sizeof(float) * h);
        break;
      }
      case kEmbedding: {
        const int64_t* ids = static_cast<const int64_t*>(P(fIn0));
        const float* table = static_cast<const float*>(P(fW));
        const float* pos = static_cast<const float*>(P(fX0));
        const long long h = r[fD0];
        const float scale = as_float(r[fScalar]);
        if (!table || !pos) return -(i + 1);
#pragma omp parallel for schedule(static)
        for (long long row = 0; row < lead; ++row) {
          float* o = out + row * h;
          const int64_t id = ids[row];
          if (id == r[fD2]) {
            std::memset(o, 0, sizeof(float) * h);
            continue;
          }
          const float* e = table + id * h;
          const float* p = pos + (step + row % seq) * h;
          for (long long j = 0; j < h; ++j) o[j] = e[j] * scale + p[j];
        }
        break;
      }
      case kAttention:
      case kCachedAttention: {
        const long long heads = r[fD1], hd = r[fD2], hidden = heads * hd;
        const bool cached = r[fOp] == kCachedAttention;
        float* kc = cached ? static_cast<float*>(P(fX0)) : nullptr;
        float* vc = cached ? static_cast<float*>(P(fX1)) : nullptr;
        const long long max_len = r[fMaxLen];
        if (cached && (!kc || !vc || step + seq > max_len)) return -(i + 1);
        const bool causal = cached || (r[fFlags] & 1);
#pragma omp parallel
        {
          std::vector<float> scores(static_cast<size_t>(max_keys));
#pragma omp for collapse(2) schedule(static)
          for (long long b = 0; b < batch; ++b) {
            for (long long hh = 0; hh < heads; ++hh) {
              const float* base = in0 + b * seq * 3 * hidden + hh * hd;  // [s, 3, heads, hd]
              const float* q = base;
              float* o = out + b * seq * hidden + hh * hd;
              const uint8_t* kp = pad ? pad + b * seq : nullptr;
              if (!cached) {
                attend(q, 3 * hidden, base + hidden, 3 * hidden, base + 2 * hidden, 3 * hidden, o, hidden, seq, seq, hd, causal, 0,
                       kp, scores.data());
              } else {
                float* kb = kc + (b * heads + hh) * max_len * hd;
                float* vb = vc + (b * heads + hh) * max_len * hd;
                for (long long t = 0; t < seq; ++t) {
                  std::memcpy(kb + (step + t) * hd, base + hidden + t * 3 * hidden, sizeof(float) * hd);
                  std::memcpy(vb + (step + t) * hd, base + 2 * hidden + t * 3 * hidden, sizeof(float) * hd);
                }
                attend(q, 3 * hidden, kb, hd, vb, hd, o, hidden, seq, step + seq, hd, true, step, nullptr, scores.data());
              }
            }
          }
        }
        break;
      }
      default:
        return -(i + 1);
    }
  }
  return 0;
}

extern "C" int oslo_cpu_graph_record_size() { return kRecord; }
