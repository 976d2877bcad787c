// Privacy-loss distributions of mechanisms and amplification schemes.
//
// A Pld holds the PMF for the "remove" adjacency and, when the mechanism is not symmetric, a second one for "add";
// every metric is the worst case over the two. Distributions are built by the connect-the-dots construction: the
// hockey-stick curve delta(eps) is evaluated on the loss grid and the unique pessimistic PMF supported on that grid
// that reproduces the curve at the grid points is solved in closed form.
#pragma once
#include "pmf.hpp"

#include <functional>
#include <memory>
#include <optional>

namespace opkacc {

struct Config {
  double discretization = 1e-4;
  double log_mass_truncation_bound = -50.0;
  size_t max_grid_size = 10000000;
  double tail_mass_truncation = 1e-15;
  uint64_t seed = 42;
  size_t max_conv_grid = 32768;
  double mc_resolution = 1e-5;
  double mc_failure_probability = 1e-6;

  double effective_discretization(double lo, double hi) const {
    const double range = hi - lo;
    const double grid = std::ceil(range / discretization);
    if (grid <= (double)max_grid_size) return discretization;
    int k = (int)std::ceil(std::log2(std::ceil(grid / (double)max_grid_size)));
    if (k < 1) k = 1;
    return discretization * std::ldexp(1.0, k);
  }
  // Monte-Carlo sample count needed to resolve tail masses of mc_resolution with the configured failure probability.
  size_t resolved_num_mc_samples() const {
    const double n = 2.0 * std::log(2.0 / mc_failure_probability) / (mc_resolution);
    return (size_t)std::min(5e7, std::max(1e4, std::ceil(n)));
  }
  void validate() const {
    if (!(discretization > 0)) throw std::invalid_argument("discretization must be positive");
    if (!(log_mass_truncation_bound < 0)) throw std::invalid_argument("log_mass_truncation_bound must be negative");
    if (max_grid_size < 2) throw std::invalid_argument("max_grid_size must be >= 2");
    if (!(tail_mass_truncation >= 0)) throw std::invalid_argument("tail_mass_truncation must be >= 0");
  }
};

constexpr double kMinNoiseMultiplier = 1e-6;

struct Pld {
  Pmf remove;
  std::optional<Pmf> add;
  double tail_truncation = 1e-15;
  double gaussian_nm = 0.0;        // > 0: this is exactly a Gaussian mechanism with that noise multiplier
  double gaussian_tail_mass = 0.0;
  double mc_failure = 0.0;         // probability that a Monte-Carlo estimate underlying this PLD is off
  double mc_resolution = 0.0;

  const Pmf& add_pmf() const { return add ? *add : remove; }
  bool symmetric() const { return !add.has_value(); }

  double delta_at(double eps) const {
    double d = pmf_delta(remove, eps);
    if (add) d = std::max(d, pmf_delta(*add, eps));
    return d;
  }
  double epsilon_at(double delta) const {
    double e = pmf_epsilon(remove, delta);
    if (add) e = std::max(e, pmf_epsilon(*add, delta));
    return e;
  }
  double infinity_mass() const { return std::max(remove.inf_mass, add ? add->inf_mass : 0.0); }
  double advantage() const { return delta_at(0.0); }
  // Bayes risk of the best membership test under prior = P(record present): prior * (1 - delta(ln((1-prior)/prior))).
  double risk_at(double prior) const {
    if (!(prior > 0.0 && prior < 1.0)) throw std::invalid_argument("prior must be in (0, 1)");
    const double e = std::log((1.0 - prior) / prior);
    auto one = [&](const Pmf& p) { return prior * (1.0 - pmf_delta(p, e)); };
    double r = one(remove);
    if (add) r = std::min(r, one(*add));
    return std::max(0.0, r);
  }
  // Trade-off curve: smallest type-II error at type-I error alpha (Neyman-Pearson over the loss thresholds).
  static double beta_of(const Pmf& p, double alpha) {
    // beta(alpha) = max_eps (1 - delta(eps) - e^eps * alpha), evaluated at the grid points (the curve is the convex
    // envelope of these lines).
    double best = 0.0;
    double mass_upper = p.inf_mass, mass_lower = 0.0;
    for (size_t i = p.probs.size(); i-- > 0;) {
      const double loss = p.loss_at((int64_t)i);
      const double d = mass_upper - std::exp(loss) * mass_lower;
      best = std::max(best, 1.0 - d - std::exp(loss) * alpha);
      if (p.probs[i] > 0) { mass_upper += p.probs[i]; mass_lower += p.probs[i] * std::exp(-loss); }
    }
    if (!p.probs.empty()) {
      const double loss = p.loss_at(-1);
      const double d = mass_upper - std::exp(loss) * mass_lower;
      best = std::max(best, 1.0 - d - std::exp(loss) * alpha);
    }
    return std::min(1.0 - alpha, std::max(0.0, best));
  }
  double beta_at(double alpha) const {
    if (!(alpha >= 0.0 && alpha <= 1.0)) throw std::invalid_argument("alpha must be in [0, 1]");
    double b = beta_of(remove, alpha);
    if (add) b = std::min(b, beta_of(*add, alpha));
    return b;
  }
};

inline Pld compose(const Pld& a, const Pld& b) {
  Pld o;
  o.tail_truncation = std::max(a.tail_truncation, b.tail_truncation);
  o.remove = compose(a.remove, b.remove, o.tail_truncation);
  if (a.add || b.add) o.add = compose(a.add_pmf(), b.add_pmf(), o.tail_truncation);
  o.mc_failure = 1.0 - (1.0 - a.mc_failure) * (1.0 - b.mc_failure);
  o.mc_resolution = std::max(a.mc_resolution, b.mc_resolution);
  return o;
}

inline Pld self_compose(const Pld& a, size_t count) {
  if (count == 0) throw std::invalid_argument("count must be >= 1");
  Pld o = a;
  o.gaussian_nm = 0.0;
  o.remove = self_compose(a.remove, count);
  if (a.add) o.add = self_compose(*a.add, count);
  o.mc_failure = a.mc_failure == 0.0 ? 0.0 : -std::expm1((double)count * std::log1p(-a.mc_failure));
  return o;
}

// ------------------------------------------------------------------------------------------------ connect the dots
inline Pmf ctd_from_deltas(std::vector<double> deltas, int64_t lo_idx, double h, size_t max_grid) {
  const size_t n = deltas.size();
  for (size_t i = 1; i < n; ++i)
    if (deltas[i] > deltas[i - 1]) deltas[i] = deltas[i - 1];
  std::map<int64_t, double> masses;
  if (n == 1) {
    if (1.0 - deltas[0] > 0) masses[lo_idx] = 1.0 - deltas[0];
    return Pmf::from_sparse(h, masses, deltas[0], max_grid);
  }
  const double exp_d = std::exp(h), em1 = std::expm1(h), em1n = std::expm1(-h);
  std::vector<double> pr(n, 0.0);
  auto diff = [&](size_t i) { return deltas[i] - deltas[i - 1]; };  // i >= 1
  pr[0] = (1.0 - deltas[0]) + diff(1) / em1;
  for (size_t i = 1; i + 1 < n; ++i) pr[i] = (diff(i + 1) - exp_d * diff(i)) / em1;
  pr[n - 1] = diff(n - 1) / em1n;
  double sum = 0.0;
  for (auto& p : pr) { if (p < 0) p = 0; sum += p; }
  const double inf_mass = deltas[n - 1], target = 1.0 - inf_mass;
  if (sum > 0 && sum != target) for (auto& p : pr) p *= target / sum;
  for (size_t i = 0; i < n; ++i)
    if (pr[i] > 0) masses[lo_idx + (int64_t)i] = pr[i];
  return Pmf::from_sparse(h, masses, inf_mass, max_grid);
}

template <class F>
inline std::vector<double> eval_parallel(int64_t lo, int64_t hi, double h, F&& f) {
  const size_t n = (size_t)(hi - lo + 1);
  std::vector<double> out(n);
  const size_t hw = std::max(1u, std::thread::hardware_concurrency());
  const size_t nthreads = n >= 10000 ? std::min<size_t>(hw, 16) : 1;
  auto work = [&](size_t a, size_t b) { for (size_t i = a; i < b; ++i) out[i] = f((double)(lo + (int64_t)i) * h); };
  if (nthreads == 1) { work(0, n); return out; }
  std::vector<std::thread> ts;
  const size_t chunk = (n + nthreads - 1) / nthreads;
  for (size_t t = 0; t < nthreads; ++t) ts.emplace_back(work, std::min(n, t * chunk), std::min(n, (t + 1) * chunk));
  for (auto& t : ts) t.join();
  return out;
}

template <class F>
inline Pmf discretize_curve(const Config& cfg, double eps_lo, double eps_hi, double h, F&& delta_fn) {
  const int64_t lo = (int64_t)std::floor(eps_lo / h), hi = (int64_t)std::ceil(eps_hi / h);
  auto deltas = eval_parallel(lo, hi, h, delta_fn);
  return ctd_from_deltas(std::move(deltas), lo, h, cfg.max_grid_size);
}

inline void set_budgets(Pld& p, const Config& cfg) {
  const double b = cfg.tail_mass_truncation / 2.0;
  p.tail_truncation = cfg.tail_mass_truncation;
  p.remove.right_budget = p.remove.left_budget = b;
  p.remove.max_grid = cfg.max_grid_size;
  if (p.add) { p.add->right_budget = p.add->left_budget = b; p.add->max_grid = cfg.max_grid_size; }
}

// ------------------------------------------------------------------------------------------------ base mechanisms
inline double gaussian_eps_upper(double nm, double log_mass) {
  const double z = norm_ppf(0.5 * std::exp(log_mass));
  return (0.5 - nm * z) / (nm * nm);
}

inline Pld gaussian_pld(double nm, const Config& cfg) {
  if (!(nm >= kMinNoiseMultiplier) || !std::isfinite(nm))
    throw std::invalid_argument("noise_multiplier must be finite and >= 1e-6");
  cfg.validate();
  const double up = gaussian_eps_upper(nm, cfg.log_mass_truncation_bound);
  const double h = cfg.effective_discretization(-up, up);
  const double dt = 1.0 / nm;
  Pld p;
  p.remove = discretize_curve(cfg, -up, up, h, [dt](double e) { return gaussian_delta_at(dt, e); });
  set_budgets(p, cfg);
  p.gaussian_nm = nm;
  p.gaussian_tail_mass = 0.5 * std::exp(cfg.log_mass_truncation_bound);
  return p;
}

inline Pld eps_delta_pld(double eps, double delta, const Config& cfg) {
  if (!(eps >= 0) || !(delta >= 0 && delta <= 1)) throw std::invalid_argument("need epsilon >= 0 and delta in [0, 1]");
  cfg.validate();
  const double h = cfg.discretization;
  const int64_t k = (int64_t)std::ceil(eps / h - 1e-12);
  std::map<int64_t, double> m;
  const double ee = std::exp(eps);
  if (k == 0) m[0] = 1.0 - delta;
  else { m[k] = (1.0 - delta) * ee / (1.0 + ee); m[-k] = (1.0 - delta) / (1.0 + ee); }
  Pld p;
  p.remove = Pmf::from_sparse(h, m, delta, cfg.max_grid_size);
  set_budgets(p, cfg);
  return p;
}

inline Pld identity_pld(const Config& cfg) {
  Pld p;
  p.remove = Pmf::from_sparse(cfg.discretization, {{0, 1.0}}, 0.0, cfg.max_grid_size);
  set_budgets(p, cfg);
  return p;
}

inline Pld non_private_pld(const Config& cfg) {
  Pld p;
  p.remove = Pmf::from_sparse(cfg.discretization, {}, 1.0, cfg.max_grid_size);
  set_budgets(p, cfg);
  return p;
}

// ------------------------------------------------------------------------------------------------ Poisson subsampling
// With P the "record present" and Q the "record absent" output distribution of the base mechanism and
// M = (1-q) Q + q P:
//   remove: H_{e^eps}(M || Q) = q * H_{e^eps'}(P || Q),  e^eps' = 1 + (e^eps - 1)/q     (1 - e^eps if e^eps <= 1-q)
//   add   : H_{e^eps}(Q || M) = c * H_{e^eps''}(Q || P), c = 1 - e^eps (1-q), e^eps'' = q e^eps / c   (0 if c <= 0)
inline Pld poisson_pld(const Pld& base, double q, const Config& cfg) {
  if (!(q > 0.0 && q <= 1.0)) throw std::invalid_argument("rate must be in (0, 1]");
  if (q == 1.0) return base;
  std::function<double(double)> d_pq, d_qp;
  double b_lo, b_hi;
  if (base.gaussian_nm > 0) {
    const double dt = 1.0 / base.gaussian_nm;
    d_pq = d_qp = [dt](double e) { return gaussian_delta_at(dt, e); };
    b_hi = gaussian_eps_upper(base.gaussian_nm, cfg.log_mass_truncation_bound);
    b_lo = -b_hi;
  } else {
    const Pmf& r = base.remove;
    const Pmf& a = base.add_pmf();
    d_pq = [&r](double e) { return pmf_delta(r, e); };
    d_qp = [&a](double e) { return pmf_delta(a, e); };
    if (r.probs.empty()) { b_lo = b_hi = 0.0; }
    else {
      b_lo = std::min(r.loss_at(0), a.probs.empty() ? 0.0 : a.loss_at(0));
      b_hi = std::max(r.loss_at((int64_t)r.size() - 1), a.probs.empty() ? 0.0 : a.loss_at((int64_t)a.size() - 1));
    }
  }
  const double r_lo = std::log1p(-q + q * std::exp(b_lo)), r_hi = std::log1p(q * std::expm1(b_hi));
  const double lo_a = -r_hi, hi_a = -r_lo;   // log dQ/dM = -log((1-q) + q dP/dQ): the mirror of the remove range
  const double h = cfg.effective_discretization(std::min(r_lo, lo_a), std::max(r_hi, hi_a));
  auto rem = [&](double e) {
    const double ee = std::exp(e);
    if (ee <= 1.0 - q) return 1.0 - ee;
    const double arg = std::log1p(std::expm1(e) / q);
    return std::min(1.0, q * d_pq(arg));
  };
  auto addf = [&](double e) {
    const double c = 1.0 - std::exp(e) * (1.0 - q);
    if (c <= 0.0) return 0.0;
    const double arg = e + std::log(q) - std::log(c);
    return std::min(1.0, c * d_qp(arg));
  };
  Pld p;
  p.remove = discretize_curve(cfg, r_lo, r_hi, h, rem);
  p.add = discretize_curve(cfg, lo_a, hi_a, h, addf);
  set_budgets(p, cfg);
  p.mc_failure = base.mc_failure;
  p.mc_resolution = base.mc_resolution;
  return p;
}

// ------------------------------------------------------------------------------------------------ Gaussian mixtures
// Record contributes j units with probability w[j] before one Gaussian noise draw: P = sum_j w_j N(j, nm^2),
// Q = N(0, nm^2). The likelihood ratio is increasing in x, so both hockey-stick curves need one root each.
inline Pld mixture_gaussian_pld(const std::vector<double>& w, double nm, const Config& cfg) {
  if (!(nm >= kMinNoiseMultiplier)) throw std::invalid_argument("noise_multiplier must be >= 1e-6");
  const int J = (int)w.size() - 1;
  const double s2 = nm * nm;
  auto log_lr = [&](double x) {
    double acc = -kInf;
    for (int j = 0; j <= J; ++j)
      if (w[j] > 0) acc = log_add_exp(acc, std::log(w[j]) + ((2.0 * j * x - (double)j * j) / (2.0 * s2)));
    return acc;
  };
  const double span = (double)J + nm * 40.0;
  auto root = [&](double target) {
    double lo = -span, hi = span;
    if (log_lr(lo) >= target) return lo;
    if (log_lr(hi) <= target) return hi;
    for (int it = 0; it < 200; ++it) {
      const double mid = 0.5 * (lo + hi);
      (log_lr(mid) < target ? lo : hi) = mid;
    }
    return 0.5 * (lo + hi);
  };
  auto sf = [](double z) { return 0.5 * std::erfc(z * M_SQRT1_2); };
  auto rem = [&](double e) {
    if (w[0] > 0 && e <= std::log(w[0])) return 1.0 - std::exp(e);
    const double x = root(e);
    double p = 0.0;
    for (int j = 0; j <= J; ++j) p += w[j] * sf((x - j) / nm);
    return std::min(1.0, std::max(0.0, p - std::exp(e) * sf(x / nm)));
  };
  auto addf = [&](double e) {
    if (w[0] > 0 && -e <= std::log(w[0])) return 0.0;
    const double x = root(-e);
    double p = 0.0;
    for (int j = 0; j <= J; ++j) p += w[j] * norm_cdf((x - j) / nm);
    return std::min(1.0, std::max(0.0, norm_cdf(x / nm) - std::exp(e) * p));
  };
  const double zt = -norm_ppf(0.5 * std::exp(cfg.log_mass_truncation_bound));
  const double hi = std::max(log_lr((double)J + nm * zt), 0.0), lo = std::min(log_lr(-nm * zt), 0.0);
  const double h = cfg.effective_discretization(std::min(lo, -hi), std::max(hi, -lo));
  Pld p;
  p.remove = discretize_curve(cfg, lo, hi, h, rem);
  p.add = discretize_curve(cfg, -hi, -lo, h, addf);
  set_budgets(p, cfg);
  return p;
}

inline double log_binom_pmf(size_t n, size_t k, double q) {
  return std::lgamma((double)n + 1) - std::lgamma((double)k + 1) - std::lgamma((double)(n - k) + 1) +
         (double)k * std::log(q) + (double)(n - k) * std::log1p(-q);
}

// Sum of `m` independent Poisson(q) draws of the same record before one noise addition.
inline Pld parallel_poisson_gaussian_pld(double nm, double q, size_t m, const Config& cfg) {
  if (!(q > 0 && q <= 1) || m == 0) throw std::invalid_argument("need rate in (0, 1] and microbatches > 0");
  std::vector<double> w;
  for (size_t j = 0; j <= m; ++j) {
    const double lp = q < 1 ? log_binom_pmf(m, j, q) : (j == m ? 0.0 : -kInf);
    if (j > 0 && lp < -80 && j > (size_t)(m * q) + 1) break;
    w.push_back(std::exp(lp));
  }
  double s = 0;
  for (double v : w) s += v;
  for (auto& v : w) v /= s;
  return mixture_gaussian_pld(w, nm, cfg);
}

// Poisson sampling with the batch capped at batch_size_max. Coupling with the uncapped mechanism fails only when the
// cap binds, so the uncapped PLD plus that probability as distinguishing mass is an upper bound.
inline Pld truncated_poisson_gaussian_pld(double nm, double q, size_t cap, size_t n, const Config& cfg) {
  Pld p = poisson_pld(gaussian_pld(nm, cfg), q, cfg);
  if (cap >= n) return p;
  double tail = 0.0;
  if (q >= 1.0) tail = 1.0;
  else {
    // P[Binomial(n, q) > cap], summed from the mode side that is smaller
    double acc = -kInf;
    for (size_t k = cap + 1; k <= n; ++k) {
      const double lp = log_binom_pmf(n, k, q);
      acc = log_add_exp(acc, lp);
      if (k > (size_t)(n * q) && lp < acc - 60) break;
    }
    tail = std::min(1.0, std::exp(acc));
  }
  p.remove.inf_mass = std::min(1.0, p.remove.inf_mass + tail);
  if (p.add) p.add->inf_mass = std::min(1.0, p.add->inf_mass + tail);
  return p;
}

}  // namespace opkacc
