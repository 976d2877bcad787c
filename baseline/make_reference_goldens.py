"""Writes the serialization fixtures under ``tests/fixtures/reference_golden/`` with the REFERENCE's own code.

    python baseline/make_reference_goldens.py [--accounting-src <path to packages/opake-accounting/src>]

Every object is built, advanced and serialized by the unmodified reference packages installed under ``baseline/_ref``
(``opake.serialization.state_dict``, the samplers' state dictionaries, ``save_dp_runtime_state``, the accountant's JSON
codec), on CPU. Each fixture also records what the reference produced NEXT from that state (the following batches of a
sampler, the following noise draw), so that a test can check that this build, after loading the state, continues the
same stream. ``optree`` / ``torchopt`` are the stand-ins of ``baseline/third_party_shims``; the reference's accounting
package is pure Python on top of a native module whose surface this build's C++ accountant reproduces, so that module
is registered under the reference's import name.

The fixtures are committed; this script is only needed to regenerate them.
"""
from __future__ import annotations

import argparse
import glob
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--accounting-src", default=os.path.join(HERE, "_ref", "opake-accounting"))
    ap.add_argument("--out", default=os.path.join(ROOT, "tests", "fixtures", "reference_golden"))
    a = ap.parse_args()
    sys.path[:0] = [os.path.join(HERE, "third_party_shims")] + sorted(glob.glob(os.path.join(HERE, "_ref", "opake-*")))
    if a.accounting_src not in sys.path:
        sys.path.insert(0, a.accounting_src)
    sys.path.insert(0, ROOT)
    from opake_b200.accounting._native import native

    sys.modules["opake.api.accounting.core.opake_accounting"] = native()

    import numpy as np
    import torch

    import opake.accounting as acc
    import opake.dpsgd.accounting as sgd_acc
    from opake.api.transformers.trainer._checkpoint import save_dp_runtime_state
    from opake.dpftrl.noise import band_mf_strategy, blt_strategy, mf_gaussian_noise
    from opake.dpftrl.sampling import BallsInBinsSampler, BMinSepSampler, CyclicPoissonSampler
    from opake.dpsgd.clipping import adaptive_clipped_grad, clipped_grad
    from opake.dpsgd.noise import gaussian_noise
    from opake.dpsgd.sampling import KOutOfTSampler, PoissonSampler
    from opake.optimizers import adamw
    from opake.random import fold_in, key
    from opake.serialization import state_dict
    from opake.types import clipped

    os.makedirs(a.out, exist_ok=True)
    out: dict = {}

    # ---- RngKey folding
    k = key(1234)
    out["rng"] = {"seed": 1234, "fold_str": fold_in(k, "opake.dpsgd.gaussian").seed, "fold_int": fold_in(k, 7).seed,
                  "fold_multi": fold_in(k, "opake.dpsgd.gaussian", 3).seed, "fold_neg": fold_in(k, -5).seed}

    # ---- Gaussian mechanism: state after three steps, and the fourth draw
    tmpl = {"b": torch.zeros(3), "w": torch.zeros(2, 4)}
    nf, ns = gaussian_noise(noise_multiplier=1.3, key=key(7))
    g = clipped(tmpl, max_norm=0.5)
    for _ in range(3):
        _, ns = nf(g, ns)
    sd = state_dict(ns)
    nxt, _ = nf(g, ns)
    out["gaussian_noise"] = {"state": sd, "noise_multiplier": 1.3, "max_norm": 0.5, "next": {n: t.clone() for n, t in nxt.pytree.items()},
                             "next_stddev": float(nxt.noise_stddev)}

    # ---- samplers: state after a few draws and the following batches
    data = list(range(200))

    def sampler_case(make, draws: int, follow: int):
        s = make()
        it = iter(s)
        for _ in range(draws):
            next(it)
        sd_ = dict(state_dict(s))
        return {"state": sd_, "next": [list(map(int, next(it))) for _ in range(follow)]}

    out["poisson"] = sampler_case(lambda: PoissonSampler(data, 0.05, n_steps=12, key=key(3)), 4, 3)
    out["poisson_truncated"] = sampler_case(lambda: PoissonSampler(data, 0.2, n_steps=12, truncated_batch_size=30, key=key(4)), 2, 3)
    out["k_out_of_t_block"] = sampler_case(lambda: KOutOfTSampler(data, k=2, t=8, allocation="block", key=key(5)), 3, 3)
    out["k_out_of_t_total"] = sampler_case(lambda: KOutOfTSampler(data, k=3, t=9, allocation="total", key=key(6)), 3, 3)
    out["cyclic_poisson"] = sampler_case(lambda: CyclicPoissonSampler(data, 0.3, bands=4, n_steps=12, key=key(8)), 5, 3)
    out["b_min_sep"] = sampler_case(lambda: BMinSepSampler(data, 3, 0.2, 12, key=key(9)), 4, 3)
    out["balls_in_bins"] = sampler_case(lambda: BallsInBinsSampler(data, 4, n_steps=12, key=key(10)), 6, 3)

    # ---- matrix-factorisation noise states (BLT, band) and their next correlated draw
    for name, strat, n_steps in (("mf_blt", blt_strategy(max_buffers=3), 64), ("mf_band", band_mf_strategy(bands=3), 16)):
        nf, ns = mf_gaussian_noise(tmpl, strat, n_steps=n_steps, noise_multiplier=1.0, key=key(5))
        for _ in range(2):
            _, ns = nf(g, ns)
        sd = state_dict(ns)
        nxt, _ = nf(g, ns)
        out[name] = {"state": sd, "n_steps": n_steps, "next": {n: t.clone() for n, t in nxt.pytree.items()},
                     "next_stddev": float(nxt.noise_stddev) if not hasattr(nxt.noise_stddev, "values") else None}

    # ---- clipping states
    w = {"w": torch.ones(4)}
    loss = lambda p, x: (p["w"] * x).sum() ** 2  # noqa: E731
    _, cs = clipped_grad(loss, clipping_norm=1.5, normalize_by=8.0)
    out["fixed_clip_state"] = dict(state_dict(cs))
    gfn, acs = adaptive_clipped_grad(loss, initial_clipping_norm=0.3, expected_batch_size=8, key=key(11))
    xs = torch.randn(8, 4, generator=torch.Generator().manual_seed(0))
    for _ in range(2):
        _, acs = gfn(w, xs, state=acs)
    out["adaptive_clip_state"] = {k_: (v.clone() if isinstance(v, torch.Tensor) else v) for k_, v in state_dict(acs).items()}

    # ---- optimizer state (AdamW-BC chain) after one update
    opt = adamw(lr=1e-2, weight_decay=0.01, noise_bias_correction=True)
    st = opt.init(tmpl)
    noisy, _ = gaussian_noise(noise_multiplier=1.0, key=key(12))[0](g, gaussian_noise(noise_multiplier=1.0, key=key(12))[1])
    _, st = opt.update(noisy, st, params=tmpl)
    out["adamw_bc_state"] = {k_: (v.clone() if isinstance(v, torch.Tensor) else v) for k_, v in state_dict(st).items()}

    torch.save(out, os.path.join(a.out, "states.pt"))

    # ---- accountant.json (nested {"type": ...} codec) and the epsilon the reference's Python layer reports for it
    ledger = acc.Accountant(budget=acc.epsilon_budget(3.0, delta=1e-5))
    ledger = ledger | (sgd_acc.poisson(sgd_acc.gaussian(1.1), 0.01) * 10)
    ledger = ledger | sgd_acc.gaussian(4.0)
    with open(os.path.join(a.out, "accountant.json"), "w", encoding="utf-8") as f:
        json.dump(state_dict(ledger), f, separators=(",", ":"))
    with open(os.path.join(a.out, "accountant_epsilon.json"), "w", encoding="utf-8") as f:
        json.dump({"delta": 1e-5, "epsilon": ledger.epsilon_at(1e-5)}, f)

    # ---- dp_state.pt (RuntimeCheckpoint, bundle version 8) written by the reference's own function
    nf, ns = gaussian_noise(noise_multiplier=1.3, key=key(7))
    _, cs = clipped_grad(loss, clipping_norm=1.5, normalize_by=8.0)
    smp = PoissonSampler(data, 0.05, n_steps=12, key=key(3))
    it = iter(smp)
    next(it)
    save_dp_runtime_state(os.path.join(a.out, "dp_state.pt"), clip_state=cs, noise_state=ns, sampler_state=dict(state_dict(smp)),
                          sample_rate=0.05, target_delta=1e-5, noise_multiplier=1.3, expected_steps_per_epoch=20,
                          expected_batch_size=10, total_steps=12, lr_scheduler="linear", learning_rate=5e-5, warmup_steps=0,
                          sampler_stream_key={"seed": 3, "impl": "opake_threefry_like"})
    print("wrote", sorted(os.listdir(a.out)))
    np.random.seed(0)


if __name__ == "__main__":
    main()
