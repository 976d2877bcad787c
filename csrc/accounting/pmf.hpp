// Dense privacy-loss PMF on a uniform loss grid and the privacy metrics computed from it.
//
// A PMF stores P[loss = (lower + i) * h] = probs[i] (pessimistic rounding: losses are rounded up), the mass at
// +infinity (distinguishing events) and at -infinity. Composition is a convolution; self-composition is an FFT power
// restricted to a Chernoff window, the mass outside of which is booked as infinite loss.
#pragma once
#include "numerics.hpp"

#include <map>
#include <string>

namespace opkacc {

struct Pmf {
  double h = 1e-4;                 // grid spacing
  int64_t lower = 0;               // loss index of probs[0]
  std::vector<double> probs;
  double inf_mass = 0.0;
  double neg_inf_mass = 0.0;
  size_t max_grid = std::numeric_limits<size_t>::max();
  double right_budget = 0.0;       // tail mass that a self-composition may move to +infinity
  double left_budget = 0.0;

  double loss_at(int64_t i) const { return (double)(lower + i) * h; }
  size_t size() const { return probs.size(); }

  static Pmf from_sparse(double h, const std::map<int64_t, double>& m, double inf_mass, size_t max_grid) {
    Pmf p;
    p.h = h;
    p.inf_mass = inf_mass;
    p.max_grid = max_grid;
    if (m.empty()) return p;
    p.lower = m.begin()->first;
    p.probs.assign((size_t)(m.rbegin()->first - p.lower + 1), 0.0);
    for (auto& kv : m) p.probs[(size_t)(kv.first - p.lower)] = kv.second;
    return p;
  }
};

inline int64_t floor_div(int64_t a, int64_t b) {
  int64_t q = a / b;
  if ((a % b != 0) && ((a < 0) != (b < 0))) --q;
  return q;
}

// Merge groups of `factor` grid points into one (rounded up to the coarse point above).
inline Pmf coarsen(const Pmf& p, size_t factor) {
  if (factor <= 1) return p;
  const int64_t f = (int64_t)factor;
  const int64_t aligned = floor_div(p.lower, f) * f;
  const size_t left = (size_t)(p.lower - aligned);
  const size_t total = left + p.probs.size();
  const size_t padded = (total + factor - 1) / factor * factor;
  Pmf o = p;
  o.h = p.h * (double)factor;
  o.probs.assign(padded / factor, 0.0);
  for (size_t i = 0; i < p.probs.size(); ++i) o.probs[(left + i) / factor] += p.probs[i];
  o.lower = aligned / f + 1;
  return o;
}

inline Pmf maybe_coarsen(Pmf p) {
  if (p.probs.size() <= p.max_grid) return p;
  const double ratio = std::ceil((double)p.probs.size() / (double)p.max_grid);
  int k = (int)std::ceil(std::log2(ratio));
  if (k < 1) k = 1;
  const size_t keep = p.max_grid;
  Pmf o = coarsen(p, size_t(1) << k);
  o.max_grid = keep;
  return o;
}

struct Truncated {
  size_t offset;
  std::vector<double> probs;
  double right_mass;
};

// Drop the longest prefix / suffix whose masses stay below tail/2 each; the prefix mass moves onto the first kept
// point (a larger loss: pessimistic), the suffix mass is returned and becomes infinite loss.
inline Truncated truncate_tails(const std::vector<double>& pr, double tail) {
  if (pr.empty() || tail <= 0.0) return {0, pr, 0.0};
  const double half = tail / 2.0;
  double lm = 0.0, rm = 0.0;
  size_t lt = 0, rt = 0;
  for (size_t i = 0; i < pr.size(); ++i) {
    if (lm + pr[i] > half) break;
    lm += pr[i];
    lt = i + 1;
  }
  for (size_t i = 0; i < pr.size(); ++i) {
    const double v = pr[pr.size() - 1 - i];
    if (rm + v > half) break;
    rm += v;
    rt = i + 1;
  }
  if (lt + rt >= pr.size()) return {0, pr, 0.0};
  std::vector<double> mid(pr.begin() + (long)lt, pr.end() - (long)rt);
  mid[0] += lm;
  return {lt, std::move(mid), rm};
}

inline double combine_budgets(double a, double b) { return std::max(a, b); }

inline bool align_grids(Pmf& a, Pmf& b) {
  const double hi = std::max(a.h, b.h), lo = std::min(a.h, b.h);
  if (std::fabs(hi - lo) <= 1e-10 * lo) return true;
  const double ratio = hi / lo, r = std::round(ratio);
  if (std::fabs(ratio - r) > 1e-9 * ratio) return false;
  const size_t f = (size_t)r;
  if (f == 0 || (f & (f - 1))) return false;
  if (a.h < b.h) a = coarsen(a, f);
  else b = coarsen(b, f);
  return true;
}

inline Pmf compose(Pmf a, Pmf b, double tail) {
  if (!align_grids(a, b))
    throw std::invalid_argument("discretization mismatch: " + std::to_string(a.h) + " vs " + std::to_string(b.h));
  Pmf o;
  o.h = a.h;
  o.max_grid = std::max(a.max_grid, b.max_grid);
  o.right_budget = combine_budgets(a.right_budget, b.right_budget);
  o.left_budget = combine_budgets(a.left_budget, b.left_budget);
  auto conv = convolve(a.probs, b.probs);
  Truncated t = truncate_tails(conv, tail);
  o.probs = std::move(t.probs);
  o.lower = a.lower + b.lower + (int64_t)t.offset;
  o.inf_mass = a.inf_mass + b.inf_mass - a.inf_mass * b.inf_mass + t.right_mass;
  o.neg_inf_mass = a.neg_inf_mass + b.neg_inf_mass - a.neg_inf_mass * b.neg_inf_mass;
  return maybe_coarsen(std::move(o));
}

inline double repeat_mass(double m, size_t count) { return m == 0.0 ? 0.0 : -std::expm1((double)count * std::log1p(-m)); }

// Window [lo, hi] of the count-fold sum outside of which at most (right, left) mass lies (Chernoff / MGF bounds).
inline std::pair<int64_t, int64_t> self_convolve_bounds(const std::vector<double>& pr, size_t count, double right,
                                                        double left) {
  if (pr.empty() || count == 0) return {0, 0};
  const int64_t full_hi = (int64_t)(pr.size() - 1) * (int64_t)count;
  if (count == 1 || (right <= 0.0 && left <= 0.0)) return {0, full_hi};
  double mean = 0.0, var = 0.0, tot = 0.0;
  for (size_t i = 0; i < pr.size(); ++i) { mean += pr[i] * (double)i; tot += pr[i]; }
  if (tot <= 0.0) return {0, full_hi};
  mean /= tot;
  for (size_t i = 0; i < pr.size(); ++i) var += pr[i] * ((double)i - mean) * ((double)i - mean);
  const double sd = std::sqrt(std::max(var / tot, 1e-12));
  std::vector<double> logp(pr.size());
  for (size_t i = 0; i < pr.size(); ++i) logp[i] = pr[i] > 0 ? std::log(pr[i]) : -kInf;
  auto log_mgf = [&](double t) {
    double mx = -kInf;
    for (size_t i = 0; i < pr.size(); ++i)
      if (logp[i] > -kInf) mx = std::max(mx, logp[i] + t * (double)i);
    double s = 0.0;
    for (size_t i = 0; i < pr.size(); ++i)
      if (logp[i] > -kInf) s += std::exp(logp[i] + t * (double)i - mx);
    return mx + std::log(s);
  };
  double best_hi = (double)full_hi, best_lo = 0.0;
  const int n_orders = 40;
  for (int j = 0; j < n_orders; ++j) {
    // orders from 1e-3/sd to 30/sd, log-spaced, both signs
    const double c = std::pow(10.0, -3.0 + (std::log10(30.0) + 3.0) * (double)j / (double)(n_orders - 1)) / sd;
    if (right > 0.0) {
      const double b = ((double)count * log_mgf(c) - std::log(right)) / c;
      if (std::isfinite(b)) best_hi = std::min(best_hi, std::ceil(b));
    }
    if (left > 0.0) {
      const double b = ((double)count * log_mgf(-c) - std::log(left)) / (-c);
      if (std::isfinite(b)) best_lo = std::max(best_lo, std::floor(b));
    }
  }
  int64_t lo = (int64_t)std::max(0.0, best_lo), hi = (int64_t)std::min((double)full_hi, best_hi);
  lo = std::min(lo, full_hi);
  hi = std::max(hi, lo);
  return {lo, hi};
}

inline Pmf self_compose(Pmf p, size_t count) {
  if (count == 0) throw std::invalid_argument("count must be >= 1");
  if (count == 1) return p;
  Pmf o = p;
  o.inf_mass = repeat_mass(p.inf_mass, count);
  o.neg_inf_mass = repeat_mass(p.neg_inf_mass, count);
  if (p.probs.empty()) return o;
  const double left = std::max(0.0, p.left_budget - p.neg_inf_mass), right = p.right_budget;
  auto [lo, hi] = self_convolve_bounds(p.probs, count, right, left);
  o.probs = self_convolve_window(p.probs, count, lo, hi);
  o.lower = p.lower * (int64_t)count + lo;
  o.inf_mass += right;
  o.neg_inf_mass += left;
  return maybe_coarsen(std::move(o));
}

// ------------------------------------------------------------------------------------------------ metrics
// delta(eps) = inf_mass + sum_{loss > eps} p * (1 - e^{eps - loss})
inline double pmf_delta(const Pmf& p, double eps) {
  double d = p.inf_mass;
  for (size_t i = p.probs.size(); i-- > 0;) {
    const double loss = p.loss_at((int64_t)i);
    if (loss <= eps) break;
    if (p.probs[i] > 0) d += p.probs[i] * -std::expm1(eps - loss);
  }
  return std::min(1.0, std::max(0.0, d));
}

// Smallest eps with delta(eps) <= delta (reverse scan over the support); +inf if the infinite mass alone exceeds it.
inline double pmf_epsilon(const Pmf& p, double delta) {
  if (p.inf_mass > delta) return kInf;
  double mass_upper = p.inf_mass, mass_lower = 0.0;  // sum p, sum p * e^{-loss} over losses above the cursor
  for (size_t i = p.probs.size(); i-- > 0;) {
    const double pr = p.probs[i];
    const double loss = p.loss_at((int64_t)i);
    // delta at eps = loss: mass_upper - e^{loss} * mass_lower
    if (mass_upper - std::exp(loss) * mass_lower >= delta) {
      // crossing lies above this grid point
      if (mass_lower <= 0.0) return loss;  // unreachable guard
      return std::max(0.0, std::log((mass_upper - delta) / mass_lower));
    }
    if (pr > 0) {
      mass_upper += pr;
      mass_lower += pr * std::exp(-loss);
    }
  }
  if (mass_upper <= delta) return 0.0;
  if (mass_lower <= 0.0) return kInf;
  return std::max(0.0, std::log((mass_upper - delta) / mass_lower));
}

}  // namespace opkacc
