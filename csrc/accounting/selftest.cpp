// Stand-alone exercise of the privacy-loss-distribution engine, meant to be built with
// -fsanitize=address,undefined (no Python, no pybind11): discretisation, FFT composition, self-composition,
// Poisson amplification, mixture curves and the metrics, checked against closed forms. Exit code 0 = all good.
#include <cmath>
#include <cstdio>
#include <vector>

#include "mechanisms.hpp"
#include "mf.hpp"

using namespace opkacc;

static int failures = 0;
#define CHECK(cond, ...)                                   \
  do {                                                     \
    if (!(cond)) {                                         \
      ++failures;                                          \
      std::printf("FAIL %s:%d: ", __FILE__, __LINE__);     \
      std::printf(__VA_ARGS__);                            \
      std::printf("\n");                                   \
    }                                                      \
  } while (0)

static double phi(double x) { return 0.5 * std::erfc(-x / std::sqrt(2.0)); }
static double gaussian_delta(double sigma, double eps) {
  return phi(0.5 / sigma - eps * sigma) - std::exp(eps) * phi(-0.5 / sigma - eps * sigma);
}

int main() {
  Config cfg;
  // 1. Gaussian: delta(eps) against the closed form
  const Pld g = gaussian_pld(1.3, cfg);
  for (double eps : {0.0, 0.5, 1.0, 2.0}) {
    const double want = gaussian_delta(1.3, eps);
    CHECK(std::fabs(g.delta_at(eps) - want) < 2e-4 * std::max(want, 1e-6) + 1e-7, "gaussian delta(%g) = %g, want %g", eps,
          g.delta_at(eps), want);
  }
  // 2. k-fold composition of a Gaussian is a Gaussian with sigma / sqrt(k)
  const Pld g16 = self_compose(gaussian_pld(4.0, cfg), 16);
  CHECK(std::fabs(g16.epsilon_at(1e-5) - gaussian_pld(1.0, cfg).epsilon_at(1e-5)) < 2e-2, "self-composition: %g vs %g",
        g16.epsilon_at(1e-5), gaussian_pld(1.0, cfg).epsilon_at(1e-5));
  const Pld g2 = compose(gaussian_pld(2.0, cfg), gaussian_pld(2.0, cfg));
  CHECK(std::fabs(g2.epsilon_at(1e-5) - gaussian_pld(std::sqrt(2.0), cfg).epsilon_at(1e-5)) < 2e-2, "pairwise composition");
  // 3. Poisson sampling: monotone in q, q = 1 gives the base mechanism back, generic transform equals the exact mixture
  const Pld base = gaussian_pld(1.1, cfg);
  const double e_full = poisson_pld(base, 1.0, cfg).epsilon_at(1e-5), e_base = base.epsilon_at(1e-5);
  CHECK(std::fabs(e_full - e_base) < 1e-3, "q=1: %g vs %g", e_full, e_base);
  double prev = 0.0;
  for (double q : {0.001, 0.01, 0.1, 0.5}) {
    const double e = self_compose(poisson_pld(base, q, cfg), 100).epsilon_at(1e-5);
    CHECK(e > prev, "epsilon must grow with q (q=%g: %g <= %g)", q, e, prev);
    prev = e;
  }
  const Pld mix = mixture_gaussian_pld({1.0 - 0.05, 0.05}, 1.1, cfg);
  CHECK(std::fabs(mix.delta_at(0.3) - poisson_pld(base, 0.05, cfg).delta_at(0.3)) < 1e-6, "mixture vs generic Poisson");
  // 4. metrics are consistent
  CHECK(base.advantage() == base.delta_at(0.0), "advantage");
  CHECK(base.beta_at(0.0) <= 1.0 && base.beta_at(1.0) == 0.0, "beta end points");
  CHECK(base.risk_at(0.5) <= 0.5 && base.risk_at(0.5) > 0.0, "risk");
  CHECK(identity_pld(cfg).epsilon_at(1e-9) == 0.0, "identity");
  CHECK(eps_delta_pld(1.0, 1e-6, cfg).epsilon_at(1e-5) <= 1.0 + 1e-9, "eps-delta atom");
  // 5. degenerate sizes and extreme parameters do not read or write out of bounds
  (void)self_compose(gaussian_pld(50.0, cfg), 1);
  (void)self_compose(gaussian_pld(0.3, cfg), 3).epsilon_at(1e-12);
  (void)poisson_pld(gaussian_pld(0.5, cfg), 1e-6, cfg).delta_at(0.0);
  std::printf(failures ? "%d check(s) failed\n" : "all checks passed\n", failures);
  return failures ? 1 : 0;
}
