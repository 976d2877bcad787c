// Matrix-factorisation (DP-FTRL) accounting helpers: participation-pattern sensitivities of strategy matrices,
// Toeplitz / lambda-CGD / banded-inverse-square-root coefficient utilities, balls-in-bins Gram matrices and the
// Monte-Carlo privacy-loss estimators for balls-in-bins and b-min-sep sampling.
//
// Conventions: strategy matrices C are lower-triangular n x n; a Toeplitz C is given by its first column c_0..c_{p-1}
// (C[r][i] = c_{r-i}); "min_sep = b" means two participations of a record are at least b steps apart and
// "max_participations = k" caps their number.
#pragma once
#include "mechanisms.hpp"

#include <atomic>
#include <mutex>
#include <numeric>
#include <unordered_map>

namespace opkacc {

inline int64_t minsep_true_max_participations(int64_t n, int64_t b, int64_t k) {
  if (n < 1 || b < 1) throw std::invalid_argument("n and min_sep must be >= 1");
  const int64_t fit = 1 + (n - 1) / b;
  return k > 0 ? std::min(fit, k) : fit;
}

// max over index sets with pairwise distance >= b and at most k elements (k <= 0: unbounded) of sum x_i.
inline double max_participation_for_linear_fn(const std::vector<double>& x, int64_t b, int64_t k) {
  const int64_t n = (int64_t)x.size();
  if (n == 0) return 0.0;
  if (b < 1) throw std::invalid_argument("min_sep must be >= 1");
  const int64_t kk = minsep_true_max_participations(n, b, k);
  // f[j][i]: best value with at most j picks among the first i entries
  std::vector<double> prev((size_t)n + 1, 0.0), cur((size_t)n + 1, 0.0);
  for (int64_t j = 1; j <= kk; ++j) {
    cur[0] = 0.0;
    for (int64_t i = 1; i <= n; ++i) {
      const int64_t back = std::max<int64_t>(0, i - b);
      const double take = x[(size_t)(i - 1)] + prev[(size_t)back];
      cur[(size_t)i] = std::max(cur[(size_t)(i - 1)], take);
    }
    std::swap(prev, cur);
  }
  return prev[(size_t)n];
}

inline double single_participation_sensitivity(const std::vector<double>& col_norms) {
  if (col_norms.empty()) throw std::invalid_argument("column_norms must not be empty");
  return *std::max_element(col_norms.begin(), col_norms.end());
}

// Columns that can be hit by one record are orthogonal when the band width does not exceed min_sep.
inline double banded_sensitivity(const std::vector<double>& gram_diag, int64_t b, int64_t k) {
  return std::sqrt(std::max(0.0, max_participation_for_linear_fn(gram_diag, b, k)));
}

inline double general_sensitivity_upper_bound(const std::vector<double>& G, int64_t n, int64_t b, int64_t k) {
  if ((int64_t)G.size() != n * n) throw std::invalid_argument("gram_matrix must have n*n entries");
  std::vector<double> row((size_t)n), best((size_t)n);
  for (int64_t i = 0; i < n; ++i) {
    for (int64_t j = 0; j < n; ++j) row[(size_t)j] = std::fabs(G[(size_t)(i * n + j)]);
    best[(size_t)i] = max_participation_for_linear_fn(row, b, k);
  }
  return std::sqrt(std::max(0.0, max_participation_for_linear_fn(best, b, k)));
}

inline double fixed_epoch_sensitivity(const std::vector<double>& G, int64_t n, int64_t epochs) {
  if ((int64_t)G.size() != n * n) throw std::invalid_argument("gram_matrix must have n*n entries");
  if (epochs < 1 || n % epochs) throw std::invalid_argument("epochs must divide n");
  const int64_t per = n / epochs;
  double best = 0.0;
  for (int64_t s = 0; s < per; ++s) {
    double acc = 0.0;
    for (int64_t a = 0; a < epochs; ++a)
      for (int64_t c = 0; c < epochs; ++c) acc += std::fabs(G[(size_t)((s + a * per) * n + (s + c * per))]);
    best = std::max(best, acc);
  }
  return std::sqrt(best);
}

// Buffered linear Toeplitz: c_0 = 1, c_i = sum_j scale_j * decay_j^{i-1}. Squared column norm over n rows.
inline double blt_sensitivity_squared(const std::vector<double>& decay, const std::vector<double>& scale, double n) {
  if (decay.size() != scale.size()) throw std::invalid_argument("buf_decay and output_scale differ in length");
  double s = 1.0;
  for (size_t j = 0; j < decay.size(); ++j)
    for (size_t l = 0; l < decay.size(); ++l) {
      const double r = decay[j] * decay[l];
      if (!(std::fabs(r) < 1.0)) throw std::invalid_argument("buffer decays must lie in (-1, 1)");
      const double geo = std::isinf(n) ? 1.0 / (1.0 - r) : (1.0 - std::pow(r, n - 1.0)) / (1.0 - r);
      s += scale[j] * scale[l] * geo;
    }
  return s;
}

// Worst case for non-negative non-increasing Toeplitz coefficients is participation at 0, b, 2b, ...:
// the squared norm of the sum of those columns.
inline double toeplitz_colsum_sq(const std::vector<double>& c, int64_t n, int64_t b, int64_t k,
                                 const std::vector<double>* col_scale = nullptr) {
  const int64_t kk = minsep_true_max_participations(n, b, k);
  double tot = 0.0;
  for (int64_t r = 0; r < n; ++r) {
    double s = 0.0;
    for (int64_t j = 0; j < kk; ++j) {
      const int64_t col = j * b;
      if (col > r) break;
      const int64_t d = r - col;
      if (d < (int64_t)c.size()) s += std::fabs(c[(size_t)d]) * (col_scale ? (*col_scale)[(size_t)col] : 1.0);
    }
    tot += s * s;
  }
  return tot;
}
inline double toeplitz_minsep_sensitivity_squared(const std::vector<double>& c, int64_t n, int64_t b, int64_t k) {
  if (c.empty()) throw std::invalid_argument("strategy_coef must not be empty");
  return toeplitz_colsum_sq(c, n, b, k);
}

inline std::vector<double> lambda_cgd_coefs(double lam, int64_t n) {
  if (!(lam >= 0.0 && lam < 1.0)) throw std::invalid_argument("lambda must be in [0, 1)");
  std::vector<double> c((size_t)n);
  double v = 1.0;
  for (int64_t i = 0; i < n; ++i) { c[(size_t)i] = v; v *= lam; }
  return c;
}
inline std::vector<double> toeplitz_inv_col_norms(const std::vector<double>& c, int64_t n) {
  // 1 / ||C[:, j]||, column j holds c_0 .. c_{n-1-j}
  std::vector<double> pre((size_t)n + 1, 0.0);
  for (int64_t i = 0; i < n; ++i) pre[(size_t)i + 1] = pre[(size_t)i] + (i < (int64_t)c.size() ? c[(size_t)i] * c[(size_t)i] : 0.0);
  std::vector<double> inv((size_t)n);
  for (int64_t j = 0; j < n; ++j) inv[(size_t)j] = 1.0 / std::sqrt(std::max(pre[(size_t)(n - j)], 1e-300));
  return inv;
}
inline double lambda_cgd_sensitivity_squared(double lam, int64_t n, int64_t b, int64_t k) {
  return toeplitz_colsum_sq(lambda_cgd_coefs(lam, n), n, b, k);
}
inline double lambda_cgd_normalized_sensitivity_squared(double lam, int64_t n, int64_t b, int64_t k) {
  auto c = lambda_cgd_coefs(lam, n);
  auto inv = toeplitz_inv_col_norms(c, n);
  return toeplitz_colsum_sq(c, n, b, k, &inv);
}
inline double lambda_cgd_max_column_norm(double lam, int64_t n) {
  if (lam == 0.0) return 1.0;
  return std::sqrt((1.0 - std::pow(lam, 2.0 * (double)n)) / (1.0 - lam * lam));
}

// First n entries of column 0 of C given the banded Toeplitz inverse with first column `inv`.
inline std::vector<double> bisr_strategy_coefficients(const std::vector<double>& inv, int64_t n) {
  if (inv.empty() || inv[0] == 0.0 || n <= 0) throw std::invalid_argument("invalid inverse coefficients or n");
  std::vector<double> c((size_t)n, 0.0);
  c[0] = 1.0 / inv[0];
  for (int64_t m = 1; m < n; ++m) {
    double s = 0.0;
    for (int64_t j = 1; j <= m && j < (int64_t)inv.size(); ++j) s += inv[(size_t)j] * c[(size_t)(m - j)];
    c[(size_t)m] = -s / inv[0];
  }
  return c;
}
inline double bisr_sensitivity_squared(const std::vector<double>& inv, int64_t n, int64_t b, int64_t k) {
  return toeplitz_colsum_sq(bisr_strategy_coefficients(inv, n), n, b, k);
}
inline double bisr_normalized_sensitivity_squared(const std::vector<double>& inv, int64_t n, int64_t b, int64_t k) {
  auto c = bisr_strategy_coefficients(inv, n);
  auto nv = toeplitz_inv_col_norms(c, n);
  return toeplitz_colsum_sq(c, n, b, k, &nv);
}

// Balls-in-bins Gram matrix: bins_per_epoch = b; m_i = sum over epochs e of column (b*e + i); G_ij = <m_i, m_j>.
inline std::vector<double> toeplitz_gram_matrix(const std::vector<double>& c, int64_t n, int64_t b, int64_t epochs,
                                                bool normalized) {
  if (b < 1 || n < 1) throw std::invalid_argument("n_steps and min_sep must be >= 1");
  const int64_t E = epochs > 0 ? epochs : (n + b - 1) / b;
  std::vector<double> inv;
  if (normalized) inv = toeplitz_inv_col_norms(c, n);
  std::vector<double> M((size_t)(b * n), 0.0);  // row i = m_i over the n output rows
  for (int64_t i = 0; i < b; ++i)
    for (int64_t e = 0; e < E; ++e) {
      const int64_t col = b * e + i;
      if (col >= n) break;
      const double sc = normalized ? inv[(size_t)col] : 1.0;
      for (int64_t r = col; r < n && r - col < (int64_t)c.size(); ++r) M[(size_t)(i * n + r)] += c[(size_t)(r - col)] * sc;
    }
  std::vector<double> G((size_t)(b * b));
  for (int64_t i = 0; i < b; ++i)
    for (int64_t j = i; j < b; ++j) {
      double s = 0.0;
      for (int64_t r = 0; r < n; ++r) s += M[(size_t)(i * n + r)] * M[(size_t)(j * n + r)];
      G[(size_t)(i * b + j)] = G[(size_t)(j * b + i)] = s;
    }
  return G;
}

inline double adaclip_sensitivity(double z, double sigma_b, int64_t groups) {
  if (!(z > 0) || !(sigma_b > 0) || groups < 1) throw std::invalid_argument("noise_multiplier, quantile_noise_std must be > 0 and num_groups >= 1");
  return std::sqrt(1.0 / (z * z) + (double)groups / (4.0 * sigma_b * sigma_b));
}

// ------------------------------------------------------------------------------------------------ Monte Carlo
// splitmix64 / xoshiro256** with Box-Muller: a counter-seeded generator per 1024-sample shard, so results do not
// depend on the number of worker threads.
struct Rng {
  uint64_t s[4];
  static uint64_t splitmix(uint64_t& x) {
    uint64_t z = (x += 0x9E3779B97F4A7C15ull);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
  }
  explicit Rng(uint64_t seed) { for (auto& v : s) v = splitmix(seed); }
  static uint64_t rotl(uint64_t x, int k) { return (x << k) | (x >> (64 - k)); }
  uint64_t next() {
    const uint64_t r = rotl(s[1] * 5, 7) * 9, t = s[1] << 17;
    s[2] ^= s[0]; s[3] ^= s[1]; s[1] ^= s[2]; s[0] ^= s[3]; s[2] ^= t; s[3] = rotl(s[3], 45);
    return r;
  }
  double uniform() { return ((double)(next() >> 11) + 0.5) * (1.0 / 9007199254740992.0); }
  double normal() {
    const double u = uniform(), v = uniform();
    return std::sqrt(-2.0 * std::log(u)) * std::cos(2.0 * M_PI * v);
  }
};

constexpr size_t kShard = 1024;

// Lower-triangular Cholesky factor of a small symmetric PSD matrix (jitter added when needed).
inline std::vector<double> cholesky(std::vector<double> A, int64_t b) {
  std::vector<double> L((size_t)(b * b), 0.0);
  for (int64_t i = 0; i < b; ++i)
    for (int64_t j = 0; j <= i; ++j) {
      double s = A[(size_t)(i * b + j)];
      for (int64_t t = 0; t < j; ++t) s -= L[(size_t)(i * b + t)] * L[(size_t)(j * b + t)];
      if (i == j) L[(size_t)(i * b + i)] = std::sqrt(std::max(s, 1e-14));
      else L[(size_t)(i * b + j)] = s / L[(size_t)(j * b + j)];
    }
  return L;
}

// Cholesky factor of a CYCLICALLY banded Gram matrix (packages/opake-accounting/src/amplification/balls_in_bins/
// cyclic_cholesky.rs). The Gram over bins of a Toeplitz strategy is banded modulo b: G_ij is non-zero only for
// min(|i-j|, b-|i-j|) <= p, corner blocks included. Eliminating a column couples the band rows below it and the p
// corner rows at the bottom, so L keeps the band in rows 0 .. b-p-1 (columns i-p .. i) and fills the last p rows
// densely. `lo[i]` is the first possibly non-zero column of row i; factorisation costs O(b p^2) and a product L z
// costs O(b p) instead of O(b^3) / O(b^2). A matrix without such structure (2p + 1 >= b) gets lo = 0: the dense factor.
struct CyclicCholesky {
  int64_t b = 0, p = 0;
  std::vector<double> L;        // row-major [b][b]; entries left of lo[i] are exactly zero
  std::vector<int64_t> lo;

  static int64_t cyclic_bandwidth(const std::vector<double>& G, int64_t b) {
    double dmax = 0.0;
    for (int64_t i = 0; i < b; ++i) dmax = std::max(dmax, std::fabs(G[(size_t)(i * b + i)]));
    const double tol = 1e-14 * dmax;
    int64_t p = 0;
    for (int64_t i = 0; i < b; ++i)
      for (int64_t j = 0; j < i; ++j)
        if (std::fabs(G[(size_t)(i * b + j)]) > tol) p = std::max(p, std::min(i - j, b - (i - j)));
    return p;
  }

  static CyclicCholesky factor(const std::vector<double>& G, int64_t b) {
    CyclicCholesky c;
    c.b = b;
    c.p = cyclic_bandwidth(G, b);
    const bool dense = 2 * c.p + 1 >= b;
    const int64_t n_band = dense ? 0 : b - c.p;
    c.lo.assign((size_t)b, 0);
    for (int64_t i = 0; i < n_band; ++i) c.lo[(size_t)i] = std::max<int64_t>(0, i - c.p);
    c.L.assign((size_t)(b * b), 0.0);
    for (int64_t i = 0; i < b; ++i)
      for (int64_t j = c.lo[(size_t)i]; j <= i; ++j) {
        double s = G[(size_t)(i * b + j)];
        for (int64_t t = std::max(c.lo[(size_t)i], c.lo[(size_t)j]); t < j; ++t) s -= c.L[(size_t)(i * b + t)] * c.L[(size_t)(j * b + t)];
        if (i == j) c.L[(size_t)(i * b + i)] = std::sqrt(std::max(s, 1e-14));
        else c.L[(size_t)(i * b + j)] = s / c.L[(size_t)(j * b + j)];
      }
    return c;
  }

  // y = scale * L z
  template <class Z>
  void apply(const Z* z, double scale, double* y) const {
    for (int64_t r = 0; r < b; ++r) {
      double s = 0.0;
      const double* row = &L[(size_t)(r * b)];
      for (int64_t t = lo[(size_t)r]; t <= r; ++t) s += row[t] * (double)z[t];
      y[r] = scale * s;
    }
  }
};

// Empirical PLD from privacy-loss samples of both directions (pessimistic rounding up to the grid).
inline Pld pld_from_loss_samples(const std::vector<double>& rem, const std::vector<double>& add, const Config& cfg) {
  auto build = [&](const std::vector<double>& v, double h) {
    std::map<int64_t, double> m;
    const double w = 1.0 / (double)v.size();
    double inf = 0.0;
    for (double x : v) {
      if (!std::isfinite(x)) { if (x > 0) inf += w; continue; }
      m[(int64_t)std::ceil(x / h)] += w;
    }
    return Pmf::from_sparse(h, m, inf, cfg.max_grid_size);
  };
  double lo = 0, hi = 0;
  for (double x : rem) if (std::isfinite(x)) { lo = std::min(lo, x); hi = std::max(hi, x); }
  for (double x : add) if (std::isfinite(x)) { lo = std::min(lo, x); hi = std::max(hi, x); }
  const double h = cfg.effective_discretization(lo, hi);
  Pld p;
  p.remove = build(rem, h);
  p.add = build(add, h);
  set_budgets(p, cfg);
  p.mc_failure = cfg.mc_failure_probability;
  p.mc_resolution = cfg.mc_resolution;
  return p;
}

// Projected draws for the balls-in-bins dominating pair: with Gram G = L L^T of the per-bin column sums, the record
// lands in bin J ~ Uniform(b); P = N(m_J, s^2 I) vs Q = N(0, s^2 I) and the loss depends on the output only through
// y = (<m_i, x>)_i. A corpus stores standard normal vectors z (so that y = L z scaled by sigma later) and J.
struct BnbCorpus {
  int64_t b = 0;
  std::vector<float> z;       // [n][b]
  std::vector<int32_t> bin;   // [n]
};

inline BnbCorpus make_bnb_corpus(int64_t b, size_t n, uint64_t seed) {
  BnbCorpus c;
  c.b = b;
  c.z.resize(n * (size_t)b);
  c.bin.resize(n);
  const size_t shards = (n + kShard - 1) / kShard;
  const size_t nthreads = std::min<size_t>(std::max(1u, std::thread::hardware_concurrency()), 16);
  std::atomic<size_t> next{0};
  auto work = [&]() {
    for (size_t s = next++; s < shards; s = next++) {
      Rng r(seed * 0x9E3779B97F4A7C15ull + s);
      for (size_t i = s * kShard; i < std::min(n, (s + 1) * kShard); ++i) {
        c.bin[i] = (int32_t)(r.next() % (uint64_t)b);
        for (int64_t j = 0; j < b; ++j) c.z[i * (size_t)b + (size_t)j] = (float)r.normal();
      }
    }
  };
  std::vector<std::thread> ts;
  for (size_t t = 0; t < nthreads; ++t) ts.emplace_back(work);
  for (auto& t : ts) t.join();
  return c;
}

inline Pld bnb_pld_from_corpus(const BnbCorpus& c, const std::vector<double>& G, double sigma, const Config& cfg) {
  const int64_t b = c.b;
  if ((int64_t)G.size() != b * b) throw std::invalid_argument("gram must have num_bins^2 entries");
  if (!(sigma > 0)) throw std::invalid_argument("sigma must be positive");
  const CyclicCholesky chol = CyclicCholesky::factor(G, b);
  const size_t n = c.bin.size();
  std::vector<double> rem(n), add(n);
  const double s2 = sigma * sigma, logb = std::log((double)b);
  const size_t nthreads = std::min<size_t>(std::max(1u, std::thread::hardware_concurrency()), 16);
  auto work = [&](size_t a, size_t e) {
    std::vector<double> y((size_t)b);
    for (size_t i = a; i < e; ++i) {
      // y_i = <m_i, noise> = sigma * (L z)_i
      chol.apply(&c.z[i * (size_t)b], sigma, y.data());
      const int64_t J = c.bin[i];
      // loss(x) = log mean_i exp((<m_i, x> - G_ii / 2) / s2); under P: <m_i, x> = G_iJ + y_i, under Q: y_i
      double lp = -kInf, lq = -kInf;
      for (int64_t r = 0; r < b; ++r) {
        const double g = G[(size_t)(r * b + r)];
        lp = log_add_exp(lp, (G[(size_t)(r * b + J)] + y[(size_t)r] - 0.5 * g) / s2);
        lq = log_add_exp(lq, (y[(size_t)r] - 0.5 * g) / s2);
      }
      rem[i] = lp - logb;
      add[i] = -(lq - logb);
    }
  };
  std::vector<std::thread> ts;
  const size_t chunk = (n + nthreads - 1) / nthreads;
  for (size_t t = 0; t < nthreads; ++t) ts.emplace_back(work, std::min(n, t * chunk), std::min(n, (t + 1) * chunk));
  for (auto& t : ts) t.join();
  return pld_from_loss_samples(rem, add, cfg);
}

class CorpusRegistry {
 public:
  int64_t put(BnbCorpus c) {
    std::lock_guard<std::mutex> g(mu_);
    const int64_t h = ++next_;
    store_[h] = std::make_shared<BnbCorpus>(std::move(c));
    return h;
  }
  std::shared_ptr<BnbCorpus> get(int64_t h) {
    std::lock_guard<std::mutex> g(mu_);
    auto it = store_.find(h);
    if (it == store_.end()) throw std::invalid_argument("unknown transcript corpus handle");
    return it->second;
  }
  void drop(int64_t h) {
    std::lock_guard<std::mutex> g(mu_);
    store_.erase(h);
  }

 private:
  std::mutex mu_;
  int64_t next_ = 0;
  std::unordered_map<int64_t, std::shared_ptr<BnbCorpus>> store_;
};

}  // namespace opkacc
