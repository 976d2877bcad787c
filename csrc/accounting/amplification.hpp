// Amplification engines that need more than a closed-form delta(eps) curve:
//
//   * random allocation (k uses out of t steps) as a deterministic PLD: sums of log-normal likelihood-ratio terms are
//     convolved on a GEOMETRIC grid (values e^{i*alpha}), by repeated squaring, with directed rounding so that the
//     result dominates the true privacy loss (Feldman & Shenfeld; reference: packages/opake-accounting/src/
//     amplification/random_allocation.rs:164 and pld/pmf/geom.rs:66-424);
//   * Poisson sampling with a batch-size cap as the two-component mixture of Ganesh (2025), Theorem 3.1
//     (reference: amplification/truncated_poisson.rs:41);
//   * banded matrix factorisation under warm-start b-min-sep sampling by Monte Carlo over the likelihood-ratio dynamic
//     programme of Dong & Ganesh (2026) (reference: amplification/b_min_sep/mc.rs:177-341).
#pragma once
#include "mf.hpp"

namespace opkacc {

// ===================================================================================================== geometric grid
// Distribution of a non-negative random variable S on the grid S = e^{(lower + i) * alpha}; zero_mass sits at S = 0
// (it adds nothing to a sum) and inf_mass at S = +infinity.
struct GeomPmf {
  double alpha = 1e-3;
  int64_t lower = 0;
  std::vector<double> probs;
  double zero_mass = 0.0;
  double inf_mass = 0.0;
};

// e^X for X ~ N(mu, s^2), X discretised on the alpha grid between its beta and 1 - beta quantiles.
// up = true : X is rounded up (an upper bound on e^X); the mass above the range becomes +infinity, the mass below it
//             moves onto the lowest grid point.
// up = false: X is rounded down; the mass above the range moves onto the highest grid point, the mass below becomes 0.
inline GeomPmf geom_lognormal(double mu, double s, double alpha, double beta, bool up) {
  const double z = -norm_ppf(beta);
  const int64_t lo = (int64_t)std::floor((mu - z * s) / alpha), hi = (int64_t)std::ceil((mu + z * s) / alpha);
  GeomPmf g;
  g.alpha = alpha;
  g.lower = lo;
  g.probs.assign((size_t)(hi - lo + 1), 0.0);
  auto cdf = [&](double x) { return norm_cdf((x - mu) / s); };
  auto sf = [&](double x) { return 0.5 * std::erfc((x - mu) / s * M_SQRT1_2); };
  for (int64_t i = lo; i <= hi; ++i) {
    // round up: index i collects X in ((i-1) alpha, i alpha]; round down: [i alpha, (i+1) alpha)
    const double a = (up ? (double)(i - 1) : (double)i) * alpha, b = (up ? (double)i : (double)(i + 1)) * alpha;
    const double m = (a + b) * 0.5 > mu ? sf(a) - sf(b) : cdf(b) - cdf(a);
    g.probs[(size_t)(i - lo)] = std::max(0.0, m);
  }
  if (up) {
    g.probs.front() += cdf((double)(lo - 1) * alpha);
    g.inf_mass = sf((double)hi * alpha);
  } else {
    g.probs.back() += sf((double)(hi + 1) * alpha);
    g.zero_mass = cdf((double)lo * alpha);
  }
  return g;
}

// Distribution of A + B for independent A, B on the same geometric grid. For grid points i <= j the sum
// e^{i a} + e^{j a} = e^{j a} (1 + e^{-(j-i) a}) is moved to index j + c(j - i), with c rounded up (upper bound) or
// down (lower bound). Beyond a distance D the offset c is constant, which turns the far part of the double sum into
// prefix sums: O(G * D) work instead of O(G^2).
inline GeomPmf geom_conv(const GeomPmf& A, const GeomPmf& B, bool up) {
  if (std::fabs(A.alpha - B.alpha) > 1e-12 * A.alpha) throw std::invalid_argument("geometric grids differ");
  const double alpha = A.alpha;
  GeomPmf out;
  out.alpha = alpha;
  out.inf_mass = A.inf_mass + B.inf_mass - A.inf_mass * B.inf_mass;
  const double fa = 1.0 - A.inf_mass, fb = 1.0 - B.inf_mass;   // finite parts; zero masses are part of them
  (void)fa; (void)fb;
  out.zero_mass = A.zero_mass * B.zero_mass;
  if (A.probs.empty() || B.probs.empty()) {
    const GeomPmf& k = A.probs.empty() ? B : A;
    const double z = A.probs.empty() ? A.zero_mass : B.zero_mass;
    out.lower = k.lower;
    out.probs = k.probs;
    for (auto& v : out.probs) v *= z;
    return out;
  }
  const int64_t lo = std::min(A.lower, B.lower);
  const int64_t hi = std::max(A.lower + (int64_t)A.probs.size(), B.lower + (int64_t)B.probs.size());   // exclusive
  const size_t G = (size_t)(hi - lo);
  std::vector<double> a(G, 0.0), b(G, 0.0);
  for (size_t i = 0; i < A.probs.size(); ++i) a[(size_t)(A.lower - lo) + i] = A.probs[i];
  for (size_t i = 0; i < B.probs.size(); ++i) b[(size_t)(B.lower - lo) + i] = B.probs[i];
  auto offset = [&](size_t d) {
    const double v = std::log1p(std::exp(-(double)d * alpha)) / alpha;
    return up ? (size_t)std::ceil(v - 1e-9) : (size_t)std::floor(v + 1e-9);
  };
  const size_t c_far = up ? 1 : 0;
  size_t D = 0;
  while (D < G && offset(D) != c_far) ++D;
  // (for up = true the offset is never below 1; for up = false it reaches 0 once e^{-d alpha} < e^{alpha} - 1)
  const size_t c0 = offset(0);
  const size_t Gout = G + c0 + 1;
  const size_t nthreads = std::min<size_t>(std::max(1u, std::thread::hardware_concurrency()), 16);
  std::vector<std::vector<double>> parts(nthreads, std::vector<double>(Gout, 0.0));
  std::atomic<size_t> next{0};
  auto work = [&](size_t tid) {
    auto& r = parts[tid];
    for (size_t d = next++; d < D; d = next++) {
      const size_t c = offset(d);
      double* rr = r.data() + c;
      if (d == 0) {
        for (size_t j = 0; j < G; ++j) rr[j] += a[j] * b[j];
      } else {
        for (size_t j = d; j < G; ++j) rr[j] += a[j - d] * b[j] + a[j] * b[j - d];
      }
    }
  };
  std::vector<std::thread> ts;
  for (size_t t = 0; t < nthreads; ++t) ts.emplace_back(work, t);
  for (auto& t : ts) t.join();
  std::vector<double> r(Gout, 0.0);
  for (auto& p : parts)
    for (size_t i = 0; i < Gout; ++i) r[i] += p[i];
  // far pairs (distance >= D): constant offset, prefix sums of the smaller operand
  if (D < G) {
    double pa = 0.0, pb = 0.0;
    for (size_t j = D; j < G; ++j) {
      pa += a[j - D];
      pb += b[j - D];
      r[j + c_far] += b[j] * pa + a[j] * pb;
    }
  }
  // a zero addend leaves the other operand where it is (exact)
  for (size_t j = 0; j < G; ++j) r[j] += A.zero_mass * b[j] + B.zero_mass * a[j];
  size_t first = 0, last = Gout;
  while (first < last && r[first] <= 0.0) ++first;
  while (last > first && r[last - 1] <= 0.0) --last;
  out.lower = lo + (int64_t)first;
  out.probs.assign(r.begin() + (long)first, r.begin() + (long)last);
  return out;
}

// Sum of `count` independent copies by repeated squaring.
inline GeomPmf geom_self_conv(const GeomPmf& p, size_t count, bool up) {
  if (count == 0) throw std::invalid_argument("count must be >= 1");
  GeomPmf base = p, acc;
  bool have = false;
  size_t n = count;
  while (true) {
    if (n & 1) {
      acc = have ? geom_conv(acc, base, up) : base;
      have = true;
    }
    n >>= 1;
    if (!n) break;
    base = geom_conv(base, base, up);
  }
  return acc;
}

// Privacy-loss PMF of sign * (ln S - ln t) on the uniform grid h, losses rounded up. sign = +1: S is an upper bound;
// sign = -1: S is a lower bound (then S = 0 is an infinite loss).
inline Pmf geom_to_loss_pmf(const GeomPmf& g, double t, double h, size_t max_grid, int sign) {
  std::map<int64_t, double> m;
  const double lt = std::log(t);
  for (size_t i = 0; i < g.probs.size(); ++i) {
    if (g.probs[i] <= 0.0) continue;
    const double loss = (double)sign * ((double)(g.lower + (int64_t)i) * g.alpha - lt);
    m[(int64_t)std::ceil(loss / h - 1e-12)] += g.probs[i];
  }
  double inf = sign > 0 ? g.inf_mass : g.zero_mass;
  double neg_inf = sign > 0 ? g.zero_mass : g.inf_mass;
  Pmf p = Pmf::from_sparse(h, m, std::min(1.0, inf), max_grid);
  p.neg_inf_mass = neg_inf;
  return maybe_coarsen(std::move(p));
}

// One record used in exactly one of t steps, chosen uniformly; Gaussian noise with multiplier nm in every step.
//   remove: loss = ln((e^{L_0} + sum_{i<t} e^{M_i}) / t),  L_0 ~ N(mu, s^2), M_i ~ N(-mu, s^2), mu = 1/(2 nm^2), s = 1/nm
//   add   : loss = -ln(sum_{i<=t} e^{M_i} / t)
inline Pld single_allocation_gaussian_pld(double nm, size_t t, const Config& cfg) {
  if (t == 1) return gaussian_pld(nm, cfg);
  const double mu = 0.5 / (nm * nm), s = 1.0 / nm;
  const double beta_total = std::min(0.49, std::max(1e-300, 0.5 * std::exp(cfg.log_mass_truncation_bound)));
  const double beta = std::min(0.49, std::max(1e-300, beta_total / (double)t));
  const double span = 2.0 * (-norm_ppf(beta)) * s;
  const double alpha = std::max(cfg.discretization, span / (double)std::max<size_t>(cfg.max_conv_grid, 16));
  Pld p;
  {
    const GeomPmf x = geom_lognormal(mu, s, alpha, beta, true);
    const GeomPmf y = geom_lognormal(-mu, s, alpha, beta, true);
    const GeomPmf sum = geom_conv(geom_self_conv(y, t - 1, true), x, true);
    p.remove = geom_to_loss_pmf(sum, (double)t, cfg.discretization, cfg.max_grid_size, +1);
  }
  {
    const GeomPmf y = geom_lognormal(-mu, s, alpha, beta, false);
    const GeomPmf sum = geom_self_conv(y, t, false);
    p.add = geom_to_loss_pmf(sum, (double)t, cfg.discretization, cfg.max_grid_size, -1);
  }
  if (!align_grids(p.remove, *p.add)) throw std::runtime_error("random allocation: loss grids cannot be aligned");
  set_budgets(p, cfg);
  return p;
}

// k uses out of t steps. Exact for k = 1; for k > 1 the steps are split into k blocks with one use per block, which is
// an upper bound on "any k of t" by joint convexity of the hockey-stick divergence (the blocks compose exactly).
inline Pld random_allocation_gaussian_pld(double nm, size_t t, size_t k, const Config& cfg) {
  if (!(nm > 0) || !std::isfinite(nm)) throw std::invalid_argument("noise_multiplier must be > 0");
  if (t == 0 || k == 0 || k > t) throw std::invalid_argument("need t >= 1 and k in [1, t]");
  cfg.validate();
  const size_t t_floor = t / k, n_ceil = t - t_floor * k, n_floor = k - n_ceil;
  std::optional<Pld> out;
  for (auto [rounds, steps] : {std::pair<size_t, size_t>{n_floor, t_floor}, std::pair<size_t, size_t>{n_ceil, t_floor + 1}}) {
    if (rounds == 0 || steps == 0) continue;
    Pld one = single_allocation_gaussian_pld(nm, steps, cfg);
    Pld all = rounds == 1 ? one : self_compose(one, rounds);
    out = out ? compose(*out, all) : all;
  }
  if (!out) throw std::invalid_argument("empty allocation decomposition");
  return *out;
}

// ===================================================================================================== truncated Poisson
inline double log_binom_sf(size_t n, size_t k_min, double q) {   // log P[Binomial(n, q) >= k_min]
  if (k_min == 0) return 0.0;
  if (k_min > n) return -kInf;
  double acc = -kInf;
  for (size_t k = k_min; k <= n; ++k) {
    const double lp = log_binom_pmf(n, k, q);
    acc = log_add_exp(acc, lp);
    if ((double)k > (double)n * q && lp < acc - 70.0) break;
  }
  return std::min(0.0, acc);
}

// Hockey-stick divergence at e^eps between (1-q) N(0,1) + q N(+d/2... ) pairs, replace adjacency: the record is swapped
// for another one, so the two mixtures are P = (1-q) N(0,1) + q N(d,1) and R = (1-q) N(0,1) + q N(-d,1), in units of the
// noise standard deviation (d = sensitivity / sigma). dP/dR increases with x: one root per eps.
inline double poisson_gaussian_replace_delta(double d, double q, double eps) {
  auto log_ratio = [&](double x) {
    const double a = log_add_exp(std::log1p(-q), std::log(q) + d * x - 0.5 * d * d);
    const double b = log_add_exp(std::log1p(-q), std::log(q) - d * x - 0.5 * d * d);
    return a - b;
  };
  const double span = 45.0 + d;
  double lo = -span, hi = span;
  if (log_ratio(hi) <= eps) return 0.0;
  if (log_ratio(lo) >= eps) lo = hi = -span;
  else
    for (int it = 0; it < 200; ++it) {
      const double mid = 0.5 * (lo + hi);
      (log_ratio(mid) < eps ? lo : hi) = mid;
    }
  const double x = 0.5 * (lo + hi);
  auto sf = [](double z) { return 0.5 * std::erfc(z * M_SQRT1_2); };
  const double p = (1.0 - q) * sf(x) + q * sf(x - d), r = (1.0 - q) * sf(x) + q * sf(x + d);
  return std::min(1.0, std::max(0.0, p - std::exp(eps) * r));
}

// Poisson-sampled Gaussian mechanism whose batch is cut to batch_size_max records (a uniform subset when the Poisson
// draw is larger), analysed as a mixture: with probability 1 - p_trunc the cap does not bind for the other n - 1
// records and the step is an ordinary Poisson step (the worse of the add and remove curves); with probability p_trunc
// it binds, the record's presence displaces another record (replace adjacency, doubled distance) and its conditional
// inclusion rate is q_cond.
inline Pld truncated_poisson_gaussian_pld_exact(double nm, double q, size_t cap, size_t n, const Config& cfg) {
  if (!(nm >= kMinNoiseMultiplier) || !std::isfinite(nm)) throw std::invalid_argument("noise_multiplier must be finite and >= 1e-6");
  if (!(q > 0.0 && q <= 1.0)) throw std::invalid_argument("rate must be in (0, 1]");
  if (cap == 0 || n == 0) throw std::invalid_argument("batch_size_max and dataset_size must be >= 1");
  cfg.validate();
  if (cap >= n || q >= 1.0) return q >= 1.0 && cap < n ? gaussian_pld(nm / 2.0, cfg) : poisson_pld(gaussian_pld(nm, cfg), q, cfg);
  const double p_trunc = std::exp(log_binom_sf(n - 1, cap, q));
  if (p_trunc <= 0.0) return poisson_pld(gaussian_pld(nm, cfg), q, cfg);
  const double q_cond = std::min(1.0, std::exp(log_binom_sf(n, cap + 1, q)) * (double)cap / (double)n / p_trunc);
  const double d1 = 1.0 / nm, d2 = 2.0 / nm;
  auto poisson_rem = [&](double e) {
    const double ee = std::exp(e);
    if (ee <= 1.0 - q) return 1.0 - ee;
    return std::min(1.0, q * gaussian_delta_at(d1, std::log1p(std::expm1(e) / q)));
  };
  auto poisson_add = [&](double e) {
    const double c = 1.0 - std::exp(e) * (1.0 - q);
    if (c <= 0.0) return 0.0;
    return std::min(1.0, c * gaussian_delta_at(d1, e + std::log(q) - std::log(c)));
  };
  auto curve = [&](double e) {
    const double c1 = std::max(poisson_rem(e), poisson_add(e));
    const double c2 = q_cond > 0.0 ? poisson_gaussian_replace_delta(d2, q_cond, e) : 0.0;
    return std::min(1.0, (1.0 - p_trunc) * c1 + p_trunc * c2);
  };
  // the capped component is dominated by an un-amplified Gaussian at doubled distance: that bounds the loss range
  const double up = gaussian_eps_upper(nm / 2.0, cfg.log_mass_truncation_bound);
  const double h = cfg.effective_discretization(-up, up);
  Pld p;
  p.remove = discretize_curve(cfg, -up, up, h, curve);
  set_budgets(p, cfg);
  return p;
}

// ===================================================================================================== b-min-sep Monte Carlo
// Banded matrix factorisation (first column `coef`, b = len(coef) bands) where a record takes part with probability p
// in any step that lies at least b steps after its previous participation ("b-min-sep"), started from the stationary
// ("warm") state. With y the noisy prefix the adversary sees,
//     P(y) / Q(y) = (f_1(y) + p * sum_{i=2..b} f_i(y)) / (1 + (b - 1) p),
//     f_i = (1 - p) f_{i+1} + p * exp((<c, y_{i..i+b-1}> - |c|^2 / 2) / sigma^2) * f_{i+b},   f_i = 1 for i > n.
// A corpus holds, per sample, the participation pattern and noise of the P branch and the noise of the Q branch in
// units of sigma, so that one corpus serves every sigma of a calibration.
struct MinSepCorpus {
  int64_t n = 0, b = 0;
  double p = 0.0;
  std::vector<uint8_t> x;       // [samples][n]
  std::vector<float> zeta;      // [samples][n]
  std::vector<float> eta;       // [samples][n]
  size_t samples() const { return n ? zeta.size() / (size_t)n : 0; }
};

inline MinSepCorpus make_minsep_corpus(int64_t bands, int64_t n, double p, size_t samples, uint64_t seed) {
  if (bands < 1 || n < 1 || !(p > 0.0 && p <= 1.0) || samples == 0) throw std::invalid_argument("bad b-min-sep corpus arguments");
  if (samples > (size_t)4e9 / (size_t)n) throw std::invalid_argument("sample count and horizon are too large");
  MinSepCorpus c;
  c.n = n; c.b = bands; c.p = p;
  c.x.assign(samples * (size_t)n, 0);
  c.zeta.resize(samples * (size_t)n);
  c.eta.resize(samples * (size_t)n);
  const size_t shards = (samples + kShard - 1) / kShard;
  const size_t nthreads = std::min<size_t>(std::max(1u, std::thread::hardware_concurrency()), 16);
  std::atomic<size_t> next{0};
  auto work = [&]() {
    for (size_t s = next++; s < shards; s = next++) {
      Rng r(seed * 0x9E3779B97F4A7C15ull + 0x5bd1e995ull + s);
      for (size_t i = s * kShard; i < std::min(samples, (s + 1) * kShard); ++i) {
        uint8_t* xi = c.x.data() + i * (size_t)n;
        // warm start: free with probability 1 / (1 + (b-1) p), else blocked for 1 .. b-1 more steps, uniformly
        int64_t barred = 0;
        if (bands > 1 && r.uniform() * (1.0 + (double)(bands - 1) * p) >= 1.0) barred = 1 + (int64_t)(r.next() % (uint64_t)(bands - 1));
        for (int64_t t = 0; t < n; ++t) {
          const bool take = barred == 0 && r.uniform() < p;
          xi[t] = take ? 1 : 0;
          barred = take ? bands - 1 : std::max<int64_t>(0, barred - 1);
        }
        for (int64_t t = 0; t < n; ++t) c.zeta[i * (size_t)n + (size_t)t] = (float)r.normal();
        for (int64_t t = 0; t < n; ++t) c.eta[i * (size_t)n + (size_t)t] = (float)r.normal();
      }
    }
  };
  std::vector<std::thread> ts;
  for (size_t t = 0; t < nthreads; ++t) ts.emplace_back(work);
  for (auto& t : ts) t.join();
  return c;
}

inline double minsep_log_ratio(const std::vector<double>& coef, const std::vector<double>& prefix_sq, double p, double sigma2,
                               const double* y, int64_t n, std::vector<double>& f) {
  const int64_t b = (int64_t)coef.size();
  f.assign((size_t)(n + b), 0.0);
  const double lp = std::log(p), l1p = p < 1.0 ? std::log1p(-p) : -kInf;
  for (int64_t i = n - 1; i >= 0; --i) {
    const int64_t len = std::min(b, n - i);
    double dot = 0.0;
    for (int64_t k = 0; k < len; ++k) dot += coef[(size_t)k] * y[i + k];
    const double block = (dot - 0.5 * prefix_sq[(size_t)(len - 1)]) / sigma2;
    f[(size_t)i] = log_add_exp(l1p + f[(size_t)(i + 1)], lp + block + f[(size_t)(i + b)]);
  }
  double num = f[0];
  for (int64_t i = 1; i < b; ++i) num = log_add_exp(num, lp + f[(size_t)i]);
  return num - std::log1p((double)(b - 1) * p);
}

inline Pld minsep_pld_from_corpus(const MinSepCorpus& c, const std::vector<double>& coef, double sigma, const Config& cfg) {
  if ((int64_t)coef.size() != c.b) throw std::invalid_argument("strategy_coef does not have the corpus' number of bands");
  if (!(sigma > 0)) throw std::invalid_argument("sigma must be positive");
  const int64_t n = c.n, b = c.b;
  std::vector<double> prefix_sq((size_t)b);
  double acc = 0.0;
  for (int64_t k = 0; k < b; ++k) { acc += coef[(size_t)k] * coef[(size_t)k]; prefix_sq[(size_t)k] = acc; }
  const size_t S = c.samples();
  std::vector<double> rem(S), add(S);
  const double s2 = sigma * sigma;
  const size_t nthreads = std::min<size_t>(std::max(1u, std::thread::hardware_concurrency()), 16);
  auto work = [&](size_t a0, size_t a1) {
    std::vector<double> y((size_t)n), f;
    for (size_t i = a0; i < a1; ++i) {
      const uint8_t* xi = c.x.data() + i * (size_t)n;
      for (int64_t t = 0; t < n; ++t) y[(size_t)t] = sigma * (double)c.zeta[i * (size_t)n + (size_t)t];
      for (int64_t j = 0; j < n; ++j)
        if (xi[j])
          for (int64_t k = 0; k < b && j + k < n; ++k) y[(size_t)(j + k)] += coef[(size_t)k];
      rem[i] = minsep_log_ratio(coef, prefix_sq, c.p, s2, y.data(), n, f);
      for (int64_t t = 0; t < n; ++t) y[(size_t)t] = sigma * (double)c.eta[i * (size_t)n + (size_t)t];
      add[i] = -minsep_log_ratio(coef, prefix_sq, c.p, s2, y.data(), n, f);
    }
  };
  std::vector<std::thread> ts;
  const size_t chunk = (S + nthreads - 1) / nthreads;
  for (size_t t = 0; t < nthreads; ++t) ts.emplace_back(work, std::min(S, t * chunk), std::min(S, (t + 1) * chunk));
  for (auto& t : ts) t.join();
  return pld_from_loss_samples(rem, add, cfg);
}

}  // namespace opkacc
