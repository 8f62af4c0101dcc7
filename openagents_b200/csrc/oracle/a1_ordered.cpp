// The CS336-A1 real-gradient model with a FIXED order of floating-point operations.
//
// The reference commits to parameter states and gradients by SHA-256 over the exact doubles, computed by scalar loops in a
// definite order, with its own exp and ln built from + - * / only, so that two machines agree bit for bit
// (apps/openagents.com/workers/api/src/cs336-a1-real-gradient-workload.ts: deterministic exp / ln :86-138, RMSNorm :351-405,
// forward :417-596, backward :602-784, shard gradient :816-866).  The NumPy oracle of this package computes the same mathematics with
// vectorised sums and agrees to the last place or two; to reproduce the published DIGESTS the order itself has to be kept, which
// is what this file does: every accumulation below runs in the index order the reference specifies, nothing is vectorised,
// reassociated or contracted (the host library is built without fast-math and with -ffp-contract=off).
//
// Model (d = model width, h = FFN width, v = vocabulary, T = positions): embedding -> RMSNorm -> single-head causal softmax
// attention (+ residual) -> RMSNorm -> gated FFN silu(x W1) * (x W3) W2 (+ residual) -> RMSNorm -> unembedding -> cross-entropy.
// Parameter layout: emb[v,d] g1[d] wq wk wv wo [d,d] g2[d] w1[d,h] w3[d,h] w2[h,d] g3[d] wu[d,v].
#include <cmath>
#include <cstdint>
#include <cstring>
#include <vector>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr double kLn2 = 0.6931471805599453;
constexpr double kEps = 1e-5;

// exp from a range reduction by ln 2 and 18 Taylor terms; the power of two is exact.
double det_exp(double x) {
  if (x < -700.0) return 0.0;
  if (x > 700.0) return INFINITY;
  const double k = std::floor(x / kLn2 + 0.5);
  const double r = x - k * kLn2;
  double term = 1.0, sum = 1.0;
  for (int i = 1; i <= 18; i++) {
    term = (term * r) / (double)i;
    sum += term;
  }
  return sum * std::ldexp(1.0, (int)k);
}

// ln from the binary exponent and an atanh series of the mantissa (19 odd terms).
double det_ln(double x) {
  uint64_t bits;
  std::memcpy(&bits, &x, 8);
  int e = (int)((bits >> 52) & 0x7ff) - 1023;
  double m = x / std::ldexp(1.0, e);
  if (m > 1.5) {
    m /= 2.0;
    e += 1;
  }
  const double t = (m - 1.0) / (m + 1.0), t2 = t * t;
  double term = t, sum = 0.0;
  for (int i = 1; i <= 37; i += 2) {
    sum += term / (double)i;
    term *= t2;
  }
  return (double)e * kLn2 + 2.0 * sum;
}

struct Shape {
  int d, h, v, T;
  size_t emb, g1, wq, wk, wv, wo, g2, w1, w3, w2, g3, wu, size;
  Shape(int d_, int h_, int v_, int T_) : d(d_), h(h_), v(v_), T(T_) {
    size_t o = 0;
    auto take = [&](size_t n) { size_t s = o; o += n; return s; };
    emb = take((size_t)v * d); g1 = take(d); wq = take((size_t)d * d); wk = take((size_t)d * d); wv = take((size_t)d * d); wo = take((size_t)d * d);
    g2 = take(d); w1 = take((size_t)d * h); w3 = take((size_t)d * h); w2 = take((size_t)h * d); g3 = take(d); wu = take((size_t)d * v);
    size = o;
  }
};

double rms_forward(const double* x, const double* gain, double* out, int d) {
  double ss = 0.0;
  for (int i = 0; i < d; i++) ss += x[i] * x[i];
  const double rms = std::sqrt(ss / d + kEps);
  for (int i = 0; i < d; i++) out[i] = (x[i] / rms) * gain[i];
  return rms;
}

// dx += dy*g/rms - x*dot/(d*rms^3) with dot = sum dy*g*x;  dgain += dy*x/rms
void rms_backward(const double* x, const double* gain, double rms, const double* dy, double* dx, double* dgain, int d) {
  double dot = 0.0;
  for (int i = 0; i < d; i++) dot += dy[i] * gain[i] * x[i];
  const double cubed = rms * rms * rms;
  for (int i = 0; i < d; i++) {
    dx[i] = dx[i] + (dy[i] * gain[i]) / rms - (x[i] * dot) / (d * cubed);
    dgain[i] = dgain[i] + (dy[i] * x[i]) / rms;
  }
}

// One sequence: returns the summed loss over positions; when grad != nullptr, adds loss_weight * d(loss)/d(params) into it.
double sequence_pass(const Shape& s, const double* P, const int32_t* sym, double loss_weight, double* grad) {
  const int d = s.d, h = s.h, v = s.v, T = s.T;
  const double sqrt_d = std::sqrt((double)d);
  std::vector<double> h0((size_t)T * d), n1((size_t)T * d), q((size_t)T * d), k((size_t)T * d), vv((size_t)T * d), alpha((size_t)T * T, 0.0),
      mix((size_t)T * d), h1((size_t)T * d), n2((size_t)T * d), gate_in((size_t)T * h), gate_sig((size_t)T * h), value((size_t)T * h),
      act((size_t)T * h), h2((size_t)T * d), n3((size_t)T * d), probs((size_t)T * v), rms1(T), rms2(T), rms3(T), scores(T), logits(v);
  double loss = 0.0;
  for (int p = 0; p < T; p++) {                                   // embeddings, first norm, projections
    const int tok = sym[p];
    for (int i = 0; i < d; i++) h0[(size_t)p * d + i] = P[s.emb + (size_t)tok * d + i];
    rms1[p] = rms_forward(&h0[(size_t)p * d], P + s.g1, &n1[(size_t)p * d], d);
    for (int j = 0; j < d; j++) {
      double sq = 0.0, sk = 0.0, sv = 0.0;
      for (int i = 0; i < d; i++) {
        const double a = n1[(size_t)p * d + i];
        sq += a * P[s.wq + (size_t)i * d + j];
        sk += a * P[s.wk + (size_t)i * d + j];
        sv += a * P[s.wv + (size_t)i * d + j];
      }
      q[(size_t)p * d + j] = sq;
      k[(size_t)p * d + j] = sk;
      vv[(size_t)p * d + j] = sv;
    }
  }
  for (int p = 0; p < T; p++) {
    double mx = -INFINITY;
    for (int u = 0; u <= p; u++) {
      double sc = 0.0;
      for (int i = 0; i < d; i++) sc += q[(size_t)p * d + i] * k[(size_t)u * d + i];
      sc /= sqrt_d;
      scores[u] = sc;
      if (sc > mx) mx = sc;
    }
    double total = 0.0;
    for (int u = 0; u <= p; u++) {
      const double e = det_exp(scores[u] - mx);
      alpha[(size_t)p * T + u] = e;
      total += e;
    }
    for (int u = 0; u <= p; u++) alpha[(size_t)p * T + u] = alpha[(size_t)p * T + u] / total;
    for (int i = 0; i < d; i++) {
      double sum = 0.0;
      for (int u = 0; u <= p; u++) sum += alpha[(size_t)p * T + u] * vv[(size_t)u * d + i];
      mix[(size_t)p * d + i] = sum;
    }
    for (int j = 0; j < d; j++) {
      double sum = 0.0;
      for (int i = 0; i < d; i++) sum += mix[(size_t)p * d + i] * P[s.wo + (size_t)i * d + j];
      h1[(size_t)p * d + j] = h0[(size_t)p * d + j] + sum;
    }
    rms2[p] = rms_forward(&h1[(size_t)p * d], P + s.g2, &n2[(size_t)p * d], d);
    for (int j = 0; j < h; j++) {
      double sg = 0.0, sv = 0.0;
      for (int i = 0; i < d; i++) {
        const double a = n2[(size_t)p * d + i];
        sg += a * P[s.w1 + (size_t)i * h + j];
        sv += a * P[s.w3 + (size_t)i * h + j];
      }
      const double sig = 1.0 / (1.0 + det_exp(-sg));
      gate_in[(size_t)p * h + j] = sg;
      gate_sig[(size_t)p * h + j] = sig;
      value[(size_t)p * h + j] = sv;
      act[(size_t)p * h + j] = sg * sig * sv;
    }
    for (int i = 0; i < d; i++) {
      double sum = 0.0;
      for (int j = 0; j < h; j++) sum += act[(size_t)p * h + j] * P[s.w2 + (size_t)j * d + i];
      h2[(size_t)p * d + i] = h1[(size_t)p * d + i] + sum;
    }
    rms3[p] = rms_forward(&h2[(size_t)p * d], P + s.g3, &n3[(size_t)p * d], d);
    double mxl = -INFINITY;
    for (int j = 0; j < v; j++) {
      double sum = 0.0;
      for (int i = 0; i < d; i++) sum += n3[(size_t)p * d + i] * P[s.wu + (size_t)i * v + j];
      logits[j] = sum;
      if (sum > mxl) mxl = sum;
    }
    double esum = 0.0;
    for (int j = 0; j < v; j++) {
      const double e = det_exp(logits[j] - mxl);
      probs[(size_t)p * v + j] = e;
      esum += e;
    }
    for (int j = 0; j < v; j++) probs[(size_t)p * v + j] = probs[(size_t)p * v + j] / esum;
    loss += det_ln(esum) + mxl - logits[sym[p + 1]];
  }
  if (!grad) return loss;

  std::vector<double> dh0((size_t)T * d, 0.0), dn1((size_t)T * d, 0.0), dq((size_t)T * d, 0.0), dk((size_t)T * d, 0.0), dv((size_t)T * d, 0.0);
  std::vector<double> dz(v), dn3(d), dh2(d), dh1(d), dact(h), dn2(d), dmix(d), dalpha(T);
  for (int p = T - 1; p >= 0; p--) {                              // positions from the last to the first
    const int target = sym[p + 1];
    for (int j = 0; j < v; j++) dz[j] = (probs[(size_t)p * v + j] - (j == target ? 1.0 : 0.0)) * loss_weight;
    for (int i = 0; i < d; i++) {
      double sum = 0.0;
      for (int j = 0; j < v; j++) {
        grad[s.wu + (size_t)i * v + j] = grad[s.wu + (size_t)i * v + j] + n3[(size_t)p * d + i] * dz[j];
        sum += P[s.wu + (size_t)i * v + j] * dz[j];
      }
      dn3[i] = sum;
    }
    std::fill(dh2.begin(), dh2.end(), 0.0);
    rms_backward(&h2[(size_t)p * d], P + s.g3, rms3[p], dn3.data(), dh2.data(), grad + s.g3, d);
    for (int i = 0; i < d; i++) dh1[i] = dh2[i];
    for (int j = 0; j < h; j++) {
      double sum = 0.0;
      for (int i = 0; i < d; i++) {
        grad[s.w2 + (size_t)j * d + i] = grad[s.w2 + (size_t)j * d + i] + act[(size_t)p * h + j] * dh2[i];
        sum += P[s.w2 + (size_t)j * d + i] * dh2[i];
      }
      dact[j] = sum;
    }
    std::fill(dn2.begin(), dn2.end(), 0.0);
    for (int j = 0; j < h; j++) {
      const double sig = gate_sig[(size_t)p * h + j], g = gate_in[(size_t)p * h + j];
      const double silu = g * sig;
      const double dvalue = dact[j] * silu;
      const double dgate = dact[j] * value[(size_t)p * h + j] * (sig * (1.0 + g * (1.0 - sig)));
      for (int i = 0; i < d; i++) {
        grad[s.w1 + (size_t)i * h + j] = grad[s.w1 + (size_t)i * h + j] + n2[(size_t)p * d + i] * dgate;
        grad[s.w3 + (size_t)i * h + j] = grad[s.w3 + (size_t)i * h + j] + n2[(size_t)p * d + i] * dvalue;
        dn2[i] = dn2[i] + P[s.w1 + (size_t)i * h + j] * dgate + P[s.w3 + (size_t)i * h + j] * dvalue;
      }
    }
    rms_backward(&h1[(size_t)p * d], P + s.g2, rms2[p], dn2.data(), dh1.data(), grad + s.g2, d);
    for (int i = 0; i < d; i++) dh0[(size_t)p * d + i] = dh0[(size_t)p * d + i] + dh1[i];
    for (int i = 0; i < d; i++) {
      double sum = 0.0;
      for (int j = 0; j < d; j++) {
        grad[s.wo + (size_t)i * d + j] = grad[s.wo + (size_t)i * d + j] + mix[(size_t)p * d + i] * dh1[j];
        sum += P[s.wo + (size_t)i * d + j] * dh1[j];
      }
      dmix[i] = sum;
    }
    double row_dot = 0.0;
    for (int u = 0; u <= p; u++) {
      double sum = 0.0;
      for (int i = 0; i < d; i++) sum += dmix[i] * vv[(size_t)u * d + i];
      dalpha[u] = sum;
      row_dot += alpha[(size_t)p * T + u] * sum;
    }
    for (int u = 0; u <= p; u++) {
      const double a = alpha[(size_t)p * T + u];
      const double dscore = a * (dalpha[u] - row_dot);
      for (int i = 0; i < d; i++) {
        dq[(size_t)p * d + i] = dq[(size_t)p * d + i] + (dscore * k[(size_t)u * d + i]) / sqrt_d;
        dk[(size_t)u * d + i] = dk[(size_t)u * d + i] + (dscore * q[(size_t)p * d + i]) / sqrt_d;
        dv[(size_t)u * d + i] = dv[(size_t)u * d + i] + a * dmix[i];
      }
    }
  }
  for (int p = 0; p < T; p++) {                                   // projections, first norm and embeddings, first to last
    for (int i = 0; i < d; i++) {
      double sum = 0.0;
      const double a = n1[(size_t)p * d + i];
      for (int j = 0; j < d; j++) {
        const double gq = dq[(size_t)p * d + j], gk = dk[(size_t)p * d + j], gv = dv[(size_t)p * d + j];
        grad[s.wq + (size_t)i * d + j] = grad[s.wq + (size_t)i * d + j] + a * gq;
        grad[s.wk + (size_t)i * d + j] = grad[s.wk + (size_t)i * d + j] + a * gk;
        grad[s.wv + (size_t)i * d + j] = grad[s.wv + (size_t)i * d + j] + a * gv;
        sum += P[s.wq + (size_t)i * d + j] * gq + P[s.wk + (size_t)i * d + j] * gk + P[s.wv + (size_t)i * d + j] * gv;
      }
      dn1[(size_t)p * d + i] = sum;
    }
    rms_backward(&h0[(size_t)p * d], P + s.g1, rms1[p], &dn1[(size_t)p * d], &dh0[(size_t)p * d], grad + s.g1, d);
    const int tok = sym[p];
    for (int i = 0; i < d; i++) grad[s.emb + (size_t)tok * d + i] = grad[s.emb + (size_t)tok * d + i] + dh0[(size_t)p * d + i];
  }
  return loss;
}

}  // namespace

B200_API double b200_a1_det_exp(double x) { return det_exp(x); }
B200_API double b200_a1_det_ln(double x) { return det_ln(x); }
B200_API uint64_t b200_a1_param_count(int d, int h, int v) { return Shape(d, h, v, 1).size; }

// Full-batch gradient of `n_seq` sequences (each T + 1 symbols) into grad_out (zeroed here); returns the mean loss per position.
B200_API double b200_a1_shard_gradient(int d, int h, int v, int T, const double* params, const int32_t* seqs, int n_seq, double* grad_out) {
  const Shape s(d, h, v, T);
  std::memset(grad_out, 0, s.size * sizeof(double));
  const double w = 1.0 / ((double)n_seq * (double)T);
  double total = 0.0;
  for (int i = 0; i < n_seq; i++) total += sequence_pass(s, params, seqs + (size_t)i * (T + 1), w, grad_out);
  return total * w;
}
B200_API double b200_a1_mean_loss(int d, int h, int v, int T, const double* params, const int32_t* seqs, int n_seq) {
  const Shape s(d, h, v, T);
  const double w = 1.0 / ((double)n_seq * (double)T);
  double total = 0.0;
  for (int i = 0; i < n_seq; i++) total += sequence_pass(s, params, seqs + (size_t)i * (T + 1), 1.0, nullptr);
  return total * w;
}
// next = params - (lr * (g0 + g1 + ...)) / n_shards, the shards added in order
B200_API void b200_a1_sgd_step(uint64_t n, const double* params, const double* const* grads, int n_shards, double lr, double* next) {
  for (uint64_t i = 0; i < n; i++) {
    double sum = 0.0;
    for (int g = 0; g < n_shards; g++) sum += grads[g][i];
    next[i] = params[i] - (lr * sum) / (double)n_shards;
  }
}
