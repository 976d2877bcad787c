"""Functional DP-SGD in ~40 lines: explicit state, per-example clipping, Gaussian noise, DP-aware AdamW, accounting.

Run: ``python examples/quickstart.py`` (CPU is enough). Mirrors the canonical loop of the reference's
``examples/quickstart.py:57-95``.
"""
import torch
from torch import nn

from opake_b200 import accounting as acc
from opake_b200.dpsgd import PoissonSampler, clipped_grad, gaussian_noise
from opake_b200.dpsgd import accounting as sgd_acc
from opake_b200.engine.functional import make_functional
from opake_b200.engine.random import fold_in, key
from opake_b200.optimizers import adamw, apply_updates


def main(steps: int = 30, batch: int = 64, n: int = 4096, target_eps: float = 4.0, delta: float = 1e-5):
    torch.manual_seed(0)
    x = torch.randn(n, 16)
    y = (x[:, :4].sum(-1) > 0).long()
    data = torch.utils.data.TensorDataset(x, y)
    model = nn.Sequential(nn.Linear(16, 32), nn.Tanh(), nn.Linear(32, 2))
    fmodel, params, _ = make_functional(model, disable_autograd_tracking=True, partition_trainable=True)

    def loss_fn(p, xe, ye):                                   # ONE example
        return nn.functional.cross_entropy(fmodel(p, xe[None]), ye[None])

    q = batch / n
    sigma = acc.calibrate(acc.epsilon_budget(target_eps, delta), lambda nm: sgd_acc.poisson(sgd_acc.gaussian(nm), q) * steps,
                          0.3, 50.0).param
    root = key(42)
    grad_fn, clip_state = clipped_grad(loss_fn, clipping_norm=1.0, normalize_by=batch, batch_argnums=(1, 2))
    noise_fn, noise_state = gaussian_noise(noise_multiplier=sigma, key=fold_in(root, "noise"))
    opt = adamw(1e-2, noise_bias_correction=True)
    opt_state = opt.init(params)
    ledger = acc.Accountant(acc.epsilon_budget(target_eps, delta))
    sampler = PoissonSampler(data, q, n_steps=steps, key=fold_in(root, "sampler"))
    for step, idx in enumerate(sampler):
        xb, yb = x[idx], y[idx]
        clipped, clip_state = grad_fn(params, xb, yb, state=clip_state)
        noised, noise_state = noise_fn(clipped, noise_state)
        updates, opt_state = opt.update(noised, opt_state, params=params)
        params = apply_updates(params, updates)
        ledger = ledger | sgd_acc.poisson(sgd_acc.gaussian(sigma), q)
        if step % 10 == 9:
            with torch.no_grad():
                accuracy = (fmodel(params, x).argmax(-1) == y).float().mean().item()
            print(f"step {step + 1:3d}  accuracy {accuracy:.3f}  epsilon {ledger.epsilon_at(delta):.3f}")
    return ledger.epsilon_at(delta)


if __name__ == "__main__":
    main()
