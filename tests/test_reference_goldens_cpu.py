"""State dictionaries, sampler cursors, the accountant JSON and ``dp_state.pt`` WRITTEN BY THE REFERENCE load here and
continue the same streams.

The fixtures under ``tests/fixtures/reference_golden`` were produced by the unmodified reference packages
(``baseline/make_reference_goldens.py``): each holds a serialized state and what the reference produced next from it.
"""
import glob
import json
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "fixtures", "reference_golden")
ROOT = os.path.dirname(HERE)


@pytest.fixture(scope="module")
def gold():
    return torch.load(os.path.join(GOLD, "states.pt"), weights_only=False)


def test_rng_key_folding_is_bit_exact(gold):
    from opake_b200.engine.random import fold_in, key
    k = key(gold["rng"]["seed"])
    assert fold_in(k, "opake.dpsgd.gaussian").seed == gold["rng"]["fold_str"]
    assert fold_in(k, 7).seed == gold["rng"]["fold_int"]
    assert fold_in(k, "opake.dpsgd.gaussian", 3).seed == gold["rng"]["fold_multi"]
    assert fold_in(k, -5).seed == gold["rng"]["fold_neg"]


def test_gaussian_noise_state_continues_the_reference_stream(gold):
    from opake_b200.base.serialization import from_state_dict, state_dict
    from opake_b200.dpsgd import gaussian_noise
    from opake_b200.engine.random import key
    from opake_b200.engine.types import clipped
    c = gold["gaussian_noise"]
    nf, ns = gaussian_noise(noise_multiplier=c["noise_multiplier"], key=key(0))
    ns = from_state_dict(ns, c["state"])
    assert state_dict(ns) == c["state"]
    g = clipped({"b": torch.zeros(3), "w": torch.zeros(2, 4)}, max_norm=c["max_norm"])
    out, _ = nf(g, ns)
    for name, want in c["next"].items():
        assert torch.equal(out.pytree[name], want), name          # same CPU generator, same leaf order, same scale
    assert float(out.noise_stddev) == pytest.approx(c["next_stddev"], rel=1e-12)


def _samplers():
    from opake_b200.dpftrl.sampling import BallsInBinsSampler, BMinSepSampler, CyclicPoissonSampler
    from opake_b200.dpsgd.sampling import KOutOfTSampler, PoissonSampler
    from opake_b200.engine.random import key
    data = list(range(200))
    return {
        "poisson": lambda: PoissonSampler(data, 0.05, n_steps=12, key=key(0)),
        "poisson_truncated": lambda: PoissonSampler(data, 0.2, n_steps=12, truncated_batch_size=30, key=key(0)),
        "k_out_of_t_block": lambda: KOutOfTSampler(data, k=2, t=8, allocation="block", key=key(0)),
        "k_out_of_t_total": lambda: KOutOfTSampler(data, k=3, t=9, allocation="total", key=key(0)),
        "cyclic_poisson": lambda: CyclicPoissonSampler(data, 0.3, bands=4, n_steps=12, key=key(0)),
        "b_min_sep": lambda: BMinSepSampler(data, 3, 0.2, 12, key=key(0)),
        "balls_in_bins": lambda: BallsInBinsSampler(data, 4, n_steps=12, key=key(0)),
    }


@pytest.mark.parametrize("name", ["poisson", "poisson_truncated", "k_out_of_t_block", "k_out_of_t_total", "cyclic_poisson",
                                  "b_min_sep", "balls_in_bins"])
def test_sampler_resumes_on_the_reference_cursor(gold, name):
    c = gold[name]
    s = _samplers()[name]()
    s.load_state_dict(c["state"])
    assert s.state_dict() == c["state"]                         # same keys, same values
    it = iter(s)
    assert [list(map(int, next(it))) for _ in range(len(c["next"]))] == c["next"]


@pytest.mark.parametrize("name", ["mf_blt", "mf_band"])
def test_mf_noise_state_written_by_the_reference_loads(gold, name):
    from opake_b200.base.serialization import from_state_dict
    from opake_b200.dpftrl import mf_gaussian_noise
    from opake_b200.dpftrl.strategies import BandMfStrategy, BltStrategy
    from opake_b200.engine.random import key
    from opake_b200.engine.types import clipped
    c = gold[name]
    tmpl = {"b": torch.zeros(3), "w": torch.zeros(2, 4)}
    if name == "mf_blt":
        nbuf = c["state"]["_inner_state[1][0]"].shape[0]
        strat = BltStrategy(max_buffers=3, buf_decay=tuple([0.5] * nbuf), output_scale=tuple([0.1] * nbuf))
    else:
        strat = BandMfStrategy(bands=3)
    nf, ns = mf_gaussian_noise(tmpl, strat, n_steps=c["n_steps"], noise_multiplier=1.0, key=key(0))
    ns = from_state_dict(ns, c["state"])
    assert ns._step_counter == 2 and ns._rng_key.seed == 5 and float(ns._first_max_norm) == 0.5
    out, _ = nf(clipped(tmpl, max_norm=0.5), ns)
    if name == "mf_blt":            # no buffers: the draw is the iid column, bit for bit
        for leaf, want in c["next"].items():
            assert torch.equal(out.pytree[leaf], want), leaf
    else:                           # same ring contents and the same iid column; the optimised band coefficients agree closely
        for leaf, want in c["next"].items():
            assert torch.allclose(out.pytree[leaf], want, rtol=0.05, atol=0.02), leaf


def test_clip_and_optimizer_state_keys_match(gold):
    from opake_b200.base.serialization import from_state_dict, state_dict
    from opake_b200.dpsgd import adaptive_clipped_grad, gaussian_noise
    from opake_b200.engine.random import key
    from opake_b200.engine.types import clipped
    from opake_b200.optimizers import adamw
    loss = lambda p, x: (p["w"] * x).sum() ** 2  # noqa: E731
    _, acs = adaptive_clipped_grad(loss, initial_clipping_norm=0.3, expected_batch_size=8, key=key(0))
    want = gold["adaptive_clip_state"]
    assert set(state_dict(acs)) == set(want)
    acs = from_state_dict(acs, want)
    assert state_dict(acs)["_current_clipping_norm"] == pytest.approx(want["_current_clipping_norm"])
    assert state_dict(acs)["_rng_key.seed"] == 11 and state_dict(acs)["_step"] == 2
    tmpl = {"b": torch.zeros(3), "w": torch.zeros(2, 4)}
    opt = adamw(lr=1e-2, weight_decay=0.01, noise_bias_correction=True)
    st = opt.init(tmpl)
    nf, ns = gaussian_noise(noise_multiplier=1.0, key=key(12))
    noisy, _ = nf(clipped(tmpl, max_norm=0.5), ns)
    _, st = opt.update(noisy, st, params=tmpl)
    mine = state_dict(st)
    ref = gold["adamw_bc_state"]
    assert set(mine) == set(ref), (sorted(mine), sorted(ref))
    st2 = from_state_dict(st, ref)
    for k_, v in state_dict(st2).items():
        if isinstance(v, torch.Tensor):
            assert torch.equal(v, ref[k_]), k_
        else:
            assert v == pytest.approx(ref[k_]), k_


def test_accountant_json_of_the_reference_loads_and_gives_its_epsilon():
    from opake_b200 import accounting as acc
    from opake_b200.base.serialization import from_state_dict, state_dict
    with open(os.path.join(GOLD, "accountant.json"), encoding="utf-8") as f:
        saved = json.load(f)
    with open(os.path.join(GOLD, "accountant_epsilon.json"), encoding="utf-8") as f:
        want = json.load(f)
    ledger = from_state_dict(acc.Accountant(), saved)
    assert state_dict(ledger) == saved                           # round trip through this build's codec: same JSON
    assert ledger.epsilon_at(want["delta"]) == pytest.approx(want["epsilon"], rel=1e-9)


def test_dp_state_bundle_written_by_the_reference_loads():
    from opake_b200.transformers import checkpoint as ckpt
    rt = ckpt.load_runtime(os.path.join(GOLD, "dp_state.pt"))
    assert rt.version == 8 and rt.noise_state["_rng_key.seed"] == 7 and rt.sampler_state["consumed"] == 1
    assert rt.sample_rate == 0.05 and rt.total_steps == 12 and rt.mechanism_kind == "gaussian" and rt.lr_scheduler == "linear"
    assert rt.sampler_stream_key == {"seed": 3, "impl": "opake_threefry_like"}


def test_dp_state_bundle_written_here_loads_in_the_reference(tmp_path):
    """The reverse direction needs the reference installed next to this repository (``baseline/_ref``)."""
    pkgs = sorted(glob.glob(os.path.join(ROOT, "baseline", "_ref", "opake-*")))
    if len(pkgs) < 5:
        pytest.skip("reference packages are not installed under baseline/_ref")
    from opake_b200.transformers import checkpoint as ckpt
    path = str(tmp_path / "dp_state.pt")
    ckpt.save_runtime(path, ckpt.RuntimeCheckpoint(clip_state={}, noise_state={"_step_counter": 2, "_rng_key.seed": 1, "_rng_key.impl": "x"},
                                                   sampler_state={"consumed": 2}, sample_rate=0.1, target_delta=1e-6, noise_multiplier=1.0,
                                                   expected_steps_per_epoch=10, expected_batch_size=8, total_steps=20,
                                                   mechanism_kind="gaussian"))
    code = ("import sys; sys.path[:0] = %r; sys.path.append(%r); "
            # the trainer package imports the accounting package, whose native module is not built here: this build's
            # C++ accountant has the same surface and stands in for it
            "from opake_b200.accounting._native import native; "
            "sys.modules['opake.api.accounting.core.opake_accounting'] = native(); "
            "from opake.api.transformers.trainer._checkpoint import load_dp_runtime_state as L; "
            "b = L(%r); assert b.version == 8 and b.noise_state['_step_counter'] == 2 and b.total_steps == 20; print('ok')"
            % ([os.path.join(ROOT, "baseline", "third_party_shims")] + pkgs, ROOT, path))
    import subprocess
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0 and "ok" in r.stdout, r.stderr[-2000:]
    # and this build reads its own file back
    assert ckpt.load_runtime(path).total_steps == 20
