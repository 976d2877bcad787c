// pybind11 surface of the privacy accountant (module name `_opake_accounting`). Mirrors the function set of the
// reference's native module (packages/opake-accounting/src/opake/api/accounting/core/opake_accounting.pyi); argument
// errors surface as ValueError, numerical failures as RuntimeError.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "amplification.hpp"

namespace py = pybind11;
using namespace opkacc;

namespace {

CorpusRegistry g_bnb;
std::mutex g_ms_mu;
std::unordered_map<int64_t, std::shared_ptr<MinSepCorpus>> g_ms;
int64_t g_ms_next = 0;

int64_t opt_k(const py::object& o) { return o.is_none() ? 0 : o.cast<int64_t>(); }

std::string pld_repr(const Pld& p) {
  return "Pld(grid=" + std::to_string(p.remove.size()) + ", discretization=" + std::to_string(p.remove.h) +
         ", infinity_mass=" + std::to_string(p.infinity_mass()) + (p.symmetric() ? ", symmetric" : ", asymmetric") + ")";
}

}  // namespace

PYBIND11_MODULE(_opake_accounting, m) {
  m.doc() = "Privacy-loss-distribution accountant (C++17, torch-free).";

  py::class_<Config>(m, "DiscretizationConfig")
      .def(py::init([](double d, double lm, size_t mg, double tm, uint64_t seed, size_t mcg, double res, double fail) {
             Config c;
             c.discretization = d; c.log_mass_truncation_bound = lm; c.max_grid_size = mg; c.tail_mass_truncation = tm;
             c.seed = seed; c.max_conv_grid = mcg; c.mc_resolution = res; c.mc_failure_probability = fail;
             c.validate();
             return c;
           }),
           py::arg("discretization") = 1e-4, py::arg("log_mass_truncation_bound") = -50.0,
           py::arg("max_grid_size") = 10000000, py::arg("tail_mass_truncation") = 1e-15, py::arg("seed") = 42,
           py::arg("max_conv_grid") = 32768, py::arg("mc_resolution") = 1e-5, py::arg("mc_failure_probability") = 1e-6)
      .def_property_readonly("discretization", [](const Config& c) { return c.discretization; })
      .def_property_readonly("log_mass_truncation_bound", [](const Config& c) { return c.log_mass_truncation_bound; })
      .def_property_readonly("max_grid_size", [](const Config& c) { return c.max_grid_size; })
      .def_property_readonly("tail_mass_truncation", [](const Config& c) { return c.tail_mass_truncation; })
      .def_property_readonly("seed", [](const Config& c) { return c.seed; })
      .def_property_readonly("max_conv_grid", [](const Config& c) { return c.max_conv_grid; })
      .def_property_readonly("mc_resolution", [](const Config& c) { return c.mc_resolution; })
      .def_property_readonly("mc_failure_probability", [](const Config& c) { return c.mc_failure_probability; })
      .def_property_readonly("resolved_num_mc_samples", [](const Config& c) { return c.resolved_num_mc_samples(); })
      .def("_key", [](const Config& c) {
        return py::make_tuple(c.discretization, c.log_mass_truncation_bound, c.max_grid_size, c.tail_mass_truncation,
                              c.seed, c.max_conv_grid, c.mc_resolution, c.mc_failure_probability);
      })
      .def("__eq__", [](const Config& a, const py::object& o) {
        if (!py::isinstance<Config>(o)) return false;
        const Config& b = o.cast<const Config&>();
        return a.discretization == b.discretization && a.log_mass_truncation_bound == b.log_mass_truncation_bound &&
               a.max_grid_size == b.max_grid_size && a.tail_mass_truncation == b.tail_mass_truncation &&
               a.seed == b.seed && a.max_conv_grid == b.max_conv_grid && a.mc_resolution == b.mc_resolution &&
               a.mc_failure_probability == b.mc_failure_probability;
      })
      .def("__hash__", [](const Config& c) {
        return py::hash(py::make_tuple(c.discretization, c.log_mass_truncation_bound, c.max_grid_size,
                                       c.tail_mass_truncation, c.seed, c.max_conv_grid, c.mc_resolution,
                                       c.mc_failure_probability));
      })
      .def("__repr__", [](const Config& c) {
        return "DiscretizationConfig(discretization=" + std::to_string(c.discretization) + ", max_grid_size=" +
               std::to_string(c.max_grid_size) + ")";
      });

  py::class_<Pld>(m, "Pld")
      .def("epsilon_at", [](const Pld& p, double delta) {
             if (!(delta >= 0 && delta <= 1)) throw std::invalid_argument("delta must be in [0, 1]");
             py::gil_scoped_release r;
             return p.epsilon_at(delta);
           }, py::arg("delta"))
      .def("delta_at", [](const Pld& p, double eps) { py::gil_scoped_release r; return p.delta_at(eps); }, py::arg("epsilon"))
      .def_property_readonly("infinity_mass", &Pld::infinity_mass)
      .def_property_readonly("mc_failure_probability", [](const Pld& p) { return p.mc_failure; })
      .def_property_readonly("mc_confidence", [](const Pld& p) { return 1.0 - p.mc_failure; })
      .def_property_readonly("mc_resolution", [](const Pld& p) { return p.mc_resolution; })
      .def_property_readonly("grid_size", [](const Pld& p) { return p.remove.size(); })
      .def_property_readonly("discretization", [](const Pld& p) { return p.remove.h; })
      .def_property_readonly("is_symmetric", &Pld::symmetric)
      .def("advantage", &Pld::advantage)
      .def("beta_at", &Pld::beta_at, py::arg("alpha"))
      .def("risk_at", &Pld::risk_at, py::arg("prior"))
      .def("compose", [](const Pld& a, const Pld& b) { py::gil_scoped_release r; return compose(a, b); }, py::arg("other"))
      .def("self_compose", [](const Pld& a, int64_t n) {
             if (n < 1) throw std::invalid_argument("count must be >= 1");
             py::gil_scoped_release r;
             return self_compose(a, (size_t)n);
           }, py::arg("count"))
      .def("__mul__", [](const Pld& a, int64_t n) { if (n < 1) throw std::invalid_argument("count must be >= 1"); return self_compose(a, (size_t)n); })
      .def("__rmul__", [](const Pld& a, int64_t n) { if (n < 1) throw std::invalid_argument("count must be >= 1"); return self_compose(a, (size_t)n); })
      .def("__or__", [](const Pld& a, const Pld& b) { return compose(a, b); })
      .def("__repr__", &pld_repr)
      .def("__str__", &pld_repr);

  m.attr("MIN_NOISE_MULTIPLIER") = kMinNoiseMultiplier;
  m.def("gaussian_pld", [](double nm, const Config& c) { py::gil_scoped_release r; return gaussian_pld(nm, c); },
        py::arg("noise_multiplier"), py::arg("config"));
  m.def("eps_delta_pld", &eps_delta_pld, py::arg("epsilon"), py::arg("delta"), py::arg("config"));
  m.def("identity_pld", &identity_pld, py::arg("config"));
  m.def("non_private_pld", &non_private_pld, py::arg("config"));
  m.def("poisson_pld", [](const Pld& base, double rate, const py::object& cfg) {
          Config c;
          if (!cfg.is_none()) c = cfg.cast<Config>();
          else { c.discretization = base.remove.h; c.tail_mass_truncation = base.tail_truncation; c.max_grid_size = base.remove.max_grid; }
          py::gil_scoped_release r;
          return poisson_pld(base, rate, c);
        }, py::arg("base"), py::arg("rate"), py::arg("config") = py::none());
  m.def("truncated_poisson_gaussian_pld", [](double nm, double q, int64_t cap, int64_t n, const Config& c) {
          if (cap < 1 || n < 1) throw std::invalid_argument("batch_size_max and dataset_size must be >= 1");
          py::gil_scoped_release r;
          return truncated_poisson_gaussian_pld_exact(nm, q, (size_t)cap, (size_t)n, c);
        }, py::arg("noise_multiplier"), py::arg("rate"), py::arg("batch_size_max"), py::arg("dataset_size"), py::arg("config"));
  m.def("parallel_poisson_gaussian_pld", [](double nm, double q, int64_t mb, const Config& c) {
          if (mb < 1) throw std::invalid_argument("microbatches must be > 0");
          py::gil_scoped_release r;
          return parallel_poisson_gaussian_pld(nm, q, (size_t)mb, c);
        }, py::arg("noise_multiplier"), py::arg("rate"), py::arg("microbatches"), py::arg("config"));
  m.def("random_allocation_gaussian_pld", [](double nm, int64_t t, int64_t k, const Config& c) {
          if (t < 1 || k < 1 || k > t) throw std::invalid_argument("need t >= 1 and k in [1, t]");
          py::gil_scoped_release r;
          return random_allocation_gaussian_pld(nm, (size_t)t, (size_t)k, c);
        }, py::arg("noise_multiplier"), py::arg("t"), py::arg("k"), py::arg("config"));
  m.def("balls_in_bins_gaussian_pld", [](double nm, int64_t bins, const Config& c) {
          if (bins < 2) throw std::invalid_argument("num_bins must be >= 2");
          py::gil_scoped_release r;
          return self_compose(poisson_pld(gaussian_pld(nm, c), 1.0 / (double)bins, c), (size_t)bins);
        }, py::arg("noise_multiplier"), py::arg("num_bins"), py::arg("config"));
  m.def("balls_in_bins_gaussian_pld_epochs", [](double nm, int64_t bins, int64_t epochs, const Config& c) {
          if (bins < 2 || epochs < 1) throw std::invalid_argument("num_bins must be >= 2 and num_epochs >= 1");
          py::gil_scoped_release r;
          return self_compose(poisson_pld(gaussian_pld(nm, c), 1.0 / (double)bins, c), (size_t)(bins * epochs));
        }, py::arg("noise_multiplier"), py::arg("num_bins"), py::arg("num_epochs"), py::arg("config"));

  m.def("bnb_mc_pld", [](const std::vector<double>& G, int64_t b, double sigma, const Config& c) {
          if (b < 1) throw std::invalid_argument("num_bins must be >= 1");
          py::gil_scoped_release r;
          auto corpus = make_bnb_corpus(b, c.resolved_num_mc_samples(), c.seed);
          return bnb_pld_from_corpus(corpus, G, sigma, c);
        }, py::arg("gram"), py::arg("num_bins"), py::arg("sigma"), py::arg("config"));
  m.def("register_bnb_transcript_corpus", [](const std::vector<double>& G, int64_t b, int64_t n, uint64_t seed) {
          if (b < 1 || n < 1 || (int64_t)G.size() != b * b) throw std::invalid_argument("bad corpus arguments");
          py::gil_scoped_release r;
          return g_bnb.put(make_bnb_corpus(b, (size_t)n, seed));
        }, py::arg("gram"), py::arg("num_bins"), py::arg("num_samples"), py::arg("seed"));
  m.def("drop_bnb_transcript_corpus", [](int64_t h) { g_bnb.drop(h); }, py::arg("handle"));
  m.def("bnb_pld_from_transcript_handle", [](int64_t h, const std::vector<double>& G, int64_t b, double sigma, const Config& c) {
          auto corpus = g_bnb.get(h);
          if (corpus->b != b) throw std::invalid_argument("num_bins differs from the registered corpus");
          py::gil_scoped_release r;
          return bnb_pld_from_corpus(*corpus, G, sigma, c);
        }, py::arg("handle"), py::arg("gram"), py::arg("num_bins"), py::arg("sigma"), py::arg("config"));

  m.def("bandmf_b_min_sep_warm_mc_pld", [](const std::vector<double>& coef, int64_t n, double p, double sigma, const Config& c) {
          if (coef.empty() || n < 1 || !(p > 0 && p <= 1)) throw std::invalid_argument("need strategy coefficients, n_steps >= 1 and p in (0, 1]");
          py::gil_scoped_release r;
          auto corpus = make_minsep_corpus((int64_t)coef.size(), n, p, c.resolved_num_mc_samples(), c.seed);
          return minsep_pld_from_corpus(corpus, coef, sigma, c);
        }, py::arg("strategy_coef"), py::arg("n_steps"), py::arg("p"), py::arg("sigma"), py::arg("config"));
  m.def("register_b_min_sep_transcript_corpus", [](const std::vector<double>& coef, int64_t n, double p, int64_t samples, uint64_t seed) {
          if (coef.empty() || samples < 1) throw std::invalid_argument("need strategy coefficients and num_samples >= 1");
          std::shared_ptr<MinSepCorpus> corpus;
          {
            py::gil_scoped_release r;
            corpus = std::make_shared<MinSepCorpus>(make_minsep_corpus((int64_t)coef.size(), n, p, (size_t)samples, seed));
          }
          std::lock_guard<std::mutex> g(g_ms_mu);
          g_ms[++g_ms_next] = corpus;
          return g_ms_next;
        }, py::arg("strategy_coef"), py::arg("n_steps"), py::arg("p"), py::arg("num_samples"), py::arg("seed"));
  m.def("drop_b_min_sep_transcript_corpus", [](int64_t h) { std::lock_guard<std::mutex> g(g_ms_mu); g_ms.erase(h); }, py::arg("handle"));
  m.def("bandmf_b_min_sep_pld_from_transcript_handle", [](int64_t h, const std::vector<double>& coef, double p, double sigma, const Config& c) {
          std::shared_ptr<MinSepCorpus> corpus;
          { std::lock_guard<std::mutex> g(g_ms_mu); auto it = g_ms.find(h); if (it == g_ms.end()) throw std::invalid_argument("unknown corpus handle"); corpus = it->second; }
          if (std::fabs(corpus->p - p) > 1e-12) throw std::invalid_argument("p differs from the registered corpus");
          py::gil_scoped_release r;
          return minsep_pld_from_corpus(*corpus, coef, sigma, c);
        }, py::arg("handle"), py::arg("strategy_coef"), py::arg("p"), py::arg("sigma"), py::arg("config"));

  m.def("mf_gaussian_pld", [](double nm, double sens, const Config& c) {
          if (!(nm > 0) || !(sens > 0)) throw std::invalid_argument("noise_multiplier and sensitivity must be positive");
          py::gil_scoped_release r;
          return gaussian_pld(nm / sens, c);
        }, py::arg("noise_multiplier"), py::arg("sensitivity"), py::arg("config"));
  m.def("max_participation_for_linear_fn", [](const std::vector<double>& x, int64_t b, const py::object& k) {
          return max_participation_for_linear_fn(x, b, opt_k(k));
        }, py::arg("x"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none());
  m.def("minsep_true_max_participations", [](int64_t n, int64_t b, const py::object& k) {
          return minsep_true_max_participations(n, b, opt_k(k));
        }, py::arg("n"), py::arg("min_sep"), py::arg("max_participations") = py::none());
  m.def("single_participation_sensitivity", &single_participation_sensitivity, py::arg("column_norms"));
  m.def("banded_sensitivity", [](const std::vector<double>& d, int64_t b, const py::object& k) {
          return banded_sensitivity(d, b, opt_k(k));
        }, py::arg("gram_diag"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none());
  m.def("general_sensitivity_upper_bound", [](const std::vector<double>& G, int64_t n, int64_t b, const py::object& k) {
          return general_sensitivity_upper_bound(G, n, b, opt_k(k));
        }, py::arg("gram_matrix"), py::arg("n"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none());
  m.def("fixed_epoch_sensitivity", &fixed_epoch_sensitivity, py::arg("gram_matrix"), py::arg("n"), py::arg("epochs"));
  m.def("blt_sensitivity_squared", &blt_sensitivity_squared, py::arg("buf_decay"), py::arg("output_scale"), py::arg("n"));
  m.def("toeplitz_minsep_sensitivity_squared", [](const std::vector<double>& c, int64_t n, int64_t b, const py::object& k) {
          return toeplitz_minsep_sensitivity_squared(c, n, b, opt_k(k));
        }, py::arg("strategy_coef"), py::arg("n"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none());
  m.def("lambda_cgd_sensitivity_squared", [](double lam, int64_t n, int64_t b, const py::object& k, double) {
          return lambda_cgd_sensitivity_squared(lam, n, b, opt_k(k));
        }, py::arg("lambda_"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(), py::arg("momentum") = 0.0);
  m.def("lambda_cgd_normalized_sensitivity_squared", [](double lam, int64_t n, int64_t b, const py::object& k, double) {
          return lambda_cgd_normalized_sensitivity_squared(lam, n, b, opt_k(k));
        }, py::arg("lambda_"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(), py::arg("momentum") = 0.0);
  m.def("lambda_cgd_max_column_norm", &lambda_cgd_max_column_norm, py::arg("lambda_"), py::arg("n_steps"));
  m.def("lambda_cgd_gram_matrix", [](double lam, int64_t n, int64_t b, const py::object& k, bool normalized, double) {
          return toeplitz_gram_matrix(lambda_cgd_coefs(lam, n), n, b, opt_k(k), normalized);
        }, py::arg("lambda_"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(),
        py::arg("normalized") = true, py::arg("momentum") = 0.0);
  m.def("lambda_cgd_gram_matrix_lr", [](double, double, int64_t, int64_t, const py::object&, bool, const std::vector<double>&) -> std::vector<double> {
          throw std::invalid_argument("learning-rate-weighted DP-lambda-CGD accounting is not supported: omit the schedule and recalibrate, or use BandMF/BLT");
        }, py::arg("lambda_"), py::arg("momentum"), py::arg("n_steps"), py::arg("min_sep"), py::arg("max_participations"),
        py::arg("normalized"), py::arg("lr_weights"));
  m.def("bisr_sensitivity_squared", [](const std::vector<double>& c, int64_t n, int64_t b, const py::object& k, double) {
          return bisr_sensitivity_squared(c, n, b, opt_k(k));
        }, py::arg("coefficients"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(), py::arg("momentum") = 0.0);
  m.def("bisr_normalized_sensitivity_squared", [](const std::vector<double>& c, int64_t n, int64_t b, const py::object& k, double) {
          return bisr_normalized_sensitivity_squared(c, n, b, opt_k(k));
        }, py::arg("coefficients"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(), py::arg("momentum") = 0.0);
  m.def("bisr_gram_matrix", [](const std::vector<double>& c, int64_t n, int64_t b, const py::object& k, bool normalized, double) {
          return toeplitz_gram_matrix(bisr_strategy_coefficients(c, n), n, b, opt_k(k), normalized);
        }, py::arg("coefficients"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(),
        py::arg("normalized") = true, py::arg("momentum") = 0.0);
  // The reference's learning-rate-weighted Gram functions are compatibility tombstones that raise ValueError on every
  // call (opake_accounting.pyi:760-778 and :816-826: "Raises: ValueError: Always"); the same contract is kept here.
  m.def("bisr_gram_matrix_lr", [](const std::vector<double>&, double, int64_t, int64_t, const py::object&, bool, const std::vector<double>&) -> std::vector<double> {
          throw std::invalid_argument("learning-rate-weighted BISR accounting is not supported: omit the schedule and recalibrate, or use BandMF/BLT");
        }, py::arg("coefficients"), py::arg("momentum"), py::arg("n_steps"), py::arg("min_sep"), py::arg("max_participations"),
        py::arg("normalized"), py::arg("lr_weights"));
  m.def("toeplitz_gram_matrix", [](const std::vector<double>& c, int64_t n, int64_t b, const py::object& k, bool normalized) {
          return toeplitz_gram_matrix(c, n, b, opt_k(k), normalized);
        }, py::arg("strategy_coef"), py::arg("n_steps"), py::arg("min_sep") = 1, py::arg("max_participations") = py::none(),
        py::arg("normalized") = true);
  m.def("bisr_strategy_coefficients", &bisr_strategy_coefficients, py::arg("coefficients"), py::arg("n"));
  // Factor of a cyclically banded Gram matrix as the balls-in-bins sampler uses it: (cyclic bandwidth, row-major L).
  m.def("cyclic_banded_cholesky", [](const std::vector<double>& gram, int64_t b) {
          if (b < 1 || (int64_t)gram.size() != b * b) throw std::invalid_argument("gram must have num_bins^2 entries");
          const CyclicCholesky c = CyclicCholesky::factor(gram, b);
          return py::make_tuple(c.p, c.L);
        }, py::arg("gram"), py::arg("num_bins"));
  m.def("adaclip_sensitivity", &adaclip_sensitivity, py::arg("noise_multiplier"), py::arg("quantile_noise_std"), py::arg("num_groups") = 1);
}
