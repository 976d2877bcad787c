// Numerical kernels of the privacy accountant: radix-2 FFT convolution, normal CDF / quantile, log-space helpers.
// Host-only, no dependencies beyond the C++17 standard library (the accountant stays importable without torch).
#pragma once
#include <algorithm>
#include <cmath>
#include <complex>
#include <cstdint>
#include <limits>
#include <stdexcept>
#include <thread>
#include <vector>

namespace opkacc {

constexpr double kInf = std::numeric_limits<double>::infinity();

// ------------------------------------------------------------------------------------------------ normal distribution
inline double norm_cdf(double x) { return 0.5 * std::erfc(-x * M_SQRT1_2); }
inline double norm_pdf(double x) { return std::exp(-0.5 * x * x) / std::sqrt(2.0 * M_PI); }

// Quantile of the standard normal: Acklam's rational approximation polished by two Halley steps (|err| < 1e-15 in
// the bulk; tails down to p ~ 1e-300 stay accurate because the refinement works on erfc).
inline double norm_ppf(double p) {
  if (!(p > 0.0)) return -kInf;
  if (!(p < 1.0)) return kInf;
  static const double a[] = {-3.969683028665376e+01, 2.209460984245205e+02, -2.759285104469687e+02,
                             1.383577518672690e+02,  -3.066479806614716e+01, 2.506628277459239e+00};
  static const double b[] = {-5.447609879822406e+01, 1.615858368580409e+02, -1.556989798598866e+02,
                             6.680131188771972e+01,  -1.328068155288572e+01};
  static const double c[] = {-7.784894002430293e-03, -3.223964580411365e-01, -2.400758277161838e+00,
                             -2.549732539343734e+00, 4.374664141464968e+00,  2.938163982698783e+00};
  static const double d[] = {7.784695709041462e-03, 3.224671290700398e-01, 2.445134137142996e+00,
                             3.754408661907416e+00};
  const double plow = 0.02425, phigh = 1 - plow;
  double x;
  if (p < plow) {
    const double q = std::sqrt(-2 * std::log(p));
    x = (((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) /
        ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1);
  } else if (p <= phigh) {
    const double q = p - 0.5, r = q * q;
    x = (((((a[0] * r + a[1]) * r + a[2]) * r + a[3]) * r + a[4]) * r + a[5]) * q /
        (((((b[0] * r + b[1]) * r + b[2]) * r + b[3]) * r + b[4]) * r + 1);
  } else {
    const double q = std::sqrt(-2 * std::log1p(-p));
    x = -(((((c[0] * q + c[1]) * q + c[2]) * q + c[3]) * q + c[4]) * q + c[5]) /
        ((((d[0] * q + d[1]) * q + d[2]) * q + d[3]) * q + 1);
  }
  for (int it = 0; it < 2; ++it) {
    const double e = norm_cdf(x) - p;
    const double u = e / norm_pdf(x);
    x = x - u / (1 + x * u / 2);
  }
  return x;
}

// Hockey-stick divergence of N(1/sigma, 1) against N(0, 1) at e^eps (delta of the Gaussian mechanism with
// sensitivity / stddev = delta_tilde).
inline double gaussian_delta_at(double delta_tilde, double eps) {
  const double xu = 0.5 * delta_tilde - eps / delta_tilde;
  const double v = norm_cdf(xu) - std::exp(eps) * norm_cdf(xu - delta_tilde);
  return v > 0.0 ? v : 0.0;
}

// ------------------------------------------------------------------------------------------------ log-space helpers
inline double log_add_exp(double a, double b) {
  if (a == -kInf) return b;
  if (b == -kInf) return a;
  const double m = std::max(a, b);
  return m + std::log1p(std::exp(-std::fabs(a - b)));
}
inline double log1mexp(double x) {  // log(1 - e^x), x <= 0
  if (x > -M_LN2) return std::log(-std::expm1(x));
  return std::log1p(-std::exp(x));
}

// ------------------------------------------------------------------------------------------------ FFT
inline size_t next_pow2(size_t n) {
  size_t p = 1;
  while (p < n) p <<= 1;
  return p;
}

class Fft {
 public:
  explicit Fft(size_t n) : n_(n) {
    if (n == 0 || (n & (n - 1))) throw std::invalid_argument("FFT size must be a power of two");
    rev_.resize(n);
    size_t bits = 0;
    while ((size_t(1) << bits) < n) ++bits;
    for (size_t i = 0; i < n; ++i) {
      size_t r = 0;
      for (size_t b = 0; b < bits; ++b)
        if (i & (size_t(1) << b)) r |= size_t(1) << (bits - 1 - b);
      rev_[i] = r;
    }
    tw_.resize(n / 2 + 1);
    for (size_t k = 0; k <= n / 2; ++k) {
      const long double ang = -2.0L * M_PIl * (long double)k / (long double)n;
      tw_[k] = std::complex<double>((double)std::cos(ang), (double)std::sin(ang));
    }
  }
  void transform(std::vector<std::complex<double>>& a, bool inverse) const {
    for (size_t i = 0; i < n_; ++i)
      if (i < rev_[i]) std::swap(a[i], a[rev_[i]]);
    for (size_t len = 2; len <= n_; len <<= 1) {
      const size_t half = len >> 1, step = n_ / len;
      for (size_t i = 0; i < n_; i += len) {
        for (size_t j = 0; j < half; ++j) {
          std::complex<double> w = tw_[j * step];
          if (inverse) w = std::conj(w);
          const std::complex<double> u = a[i + j], v = a[i + j + half] * w;
          a[i + j] = u + v;
          a[i + j + half] = u - v;
        }
      }
    }
    if (inverse) {
      const double s = 1.0 / (double)n_;
      for (auto& x : a) x *= s;
    }
  }

 private:
  size_t n_;
  std::vector<size_t> rev_;
  std::vector<std::complex<double>> tw_;
};

constexpr size_t kMaxLinearFftSize = size_t(32) << 20;

inline void clamp_nonneg(std::vector<double>& v) {
  for (auto& x : v)
    if (!(x > 0.0)) x = 0.0;
}

// Linear convolution of two non-negative sequences.
inline std::vector<double> convolve(const std::vector<double>& x, const std::vector<double>& y) {
  if (x.empty() || y.empty()) return {};
  const size_t out = x.size() + y.size() - 1;
  if (std::min(x.size(), y.size()) <= 32) {
    std::vector<double> r(out, 0.0);
    for (size_t i = 0; i < x.size(); ++i)
      for (size_t j = 0; j < y.size(); ++j) r[i + j] += x[i] * y[j];
    return r;
  }
  const size_t n = next_pow2(out);
  Fft f(n);
  std::vector<std::complex<double>> a(n), b(n);
  for (size_t i = 0; i < x.size(); ++i) a[i] = x[i];
  for (size_t i = 0; i < y.size(); ++i) b[i] = y[i];
  f.transform(a, false);
  f.transform(b, false);
  for (size_t i = 0; i < n; ++i) a[i] *= b[i];
  f.transform(a, true);
  std::vector<double> r(out);
  for (size_t i = 0; i < out; ++i) r[i] = a[i].real();
  clamp_nonneg(r);
  return r;
}

// count-fold self convolution restricted to output indices [lo, hi] (inclusive, in units of the full result).
// The transform length only has to cover the window: mass that would alias from outside is bounded by the tail
// budgets that produced the window (Chernoff), and the caller books that mass as infinite loss.
inline std::vector<double> self_convolve_window(const std::vector<double>& x, size_t count, int64_t lo, int64_t hi) {
  const int64_t width = hi - lo + 1;
  if (width <= 0) return {};
  const size_t n = next_pow2(std::max<size_t>((size_t)width, x.size()));
  if (n > kMaxLinearFftSize * 2) throw std::runtime_error("self-composition window exceeds the FFT size limit");
  Fft f(n);
  std::vector<std::complex<double>> a(n);
  for (size_t i = 0; i < x.size(); ++i) a[i % n] += x[i];
  f.transform(a, false);
  // multiply by the phase that shifts output index `lo` to 0, then raise to the power `count`
  for (size_t k = 0; k < n; ++k) {
    const double mag = std::abs(a[k]);
    if (mag == 0.0) { a[k] = 0.0; continue; }
    const double ang = std::arg(a[k]) * (double)count + 2.0 * M_PI * (double)((k * (uint64_t)(((lo % (int64_t)n) + (int64_t)n) % (int64_t)n)) % n) / (double)n;
    a[k] = std::polar(std::pow(mag, (double)count), ang);
  }
  f.transform(a, true);
  std::vector<double> r((size_t)width);
  for (int64_t i = 0; i < width; ++i) r[(size_t)i] = a[(size_t)i].real();
  clamp_nonneg(r);
  return r;
}

}  // namespace opkacc
