"""Kernel micro-benchmarks: ``python -m benchmarks.microbench <case> [options]``.

Each case times ONE native kernel (or a short kernel sequence) in isolation with CUDA events on the launching
stream, after warm-up, writing a buffer larger than L2 between timed launches so that every launch starts cold, and
prints one JSON line per shape with the achieved rate and the fraction of the measured machine peaks
(``MEASURED_PEAKS.json`` at the repository root when present). ``--small`` shrinks the problem to a few hundred MB so
that a profiler capture of the same command ends quickly; ``--once`` runs a single launch per shape after warm-up.

Cases: ``gemm`` (forward / dgrad / wgrad shapes of a decoder layer), ``attention`` (causal GQA forward + backward),
``dp_step`` (fused noise + AdamW-BC on a parameter shard), ``clip_accumulate``, ``rmsnorm``, ``lce``, ``clip_sum``, ``moe``
(one mixture-of-experts layer on one GPU).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch


def _peaks() -> dict:
    here = os.path.dirname(os.path.abspath(__file__))
    path = os.path.join(here, "..", "MEASURED_PEAKS.json")
    try:
        with open(path, encoding="utf-8") as f:
            raw = json.load(f)
        return {"hbm_gbs": float(raw.get("hbm_gbs", 6650.0)), "bf16_tflops": float(raw.get("bf16_tflops", 1590.0)), "source": "measured"}
    except Exception:
        return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class _Timer:
    def __init__(self, device, flush_mb: int = 256):
        self.device = device
        self.flush = torch.empty(flush_mb << 20, dtype=torch.uint8, device=device)

    def run(self, fn, iters: int, warmup: int = 3) -> float:
        """Median device time of ``fn`` in microseconds, L2 flushed before every timed launch."""
        for _ in range(warmup):
            fn()
        torch.cuda.synchronize(self.device)
        times = []
        for _ in range(iters):
            self.flush.fill_(1)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize(self.device)
            times.append(a.elapsed_time(b) * 1e3)
        times.sort()
        return times[len(times) // 2]


def _emit(case: str, shape: dict, us: float, *, flops: float = 0.0, bytes_: float = 0.0) -> None:
    pk = _peaks()
    rec = {"case": case, **shape, "us": round(us, 2)}
    if flops:
        rec["tflops"] = round(flops / us * 1e-6, 1)
        rec["frac_of_bf16_peak"] = round(flops / us * 1e-6 / pk["bf16_tflops"], 3)
    if bytes_:
        rec["gbs"] = round(bytes_ / us * 1e-3, 1)
        rec["frac_of_hbm_peak"] = round(bytes_ / us * 1e-3 / pk["hbm_gbs"], 3)
    rec["peaks"] = pk["source"]
    print(json.dumps(rec), flush=True)


def case_gemm(t: _Timer, a) -> None:
    from opake_b200.ops import gemm as G
    dev = t.device
    T = 1024 if a.small else 2048
    d, f, qkv = (2048, 8192, 3072) if a.small else (4096, 14336, 6144)
    bf = torch.bfloat16
    shapes = [("fwd_qkv", T, qkv, d), ("fwd_gate_up", T, 2 * f, d), ("fwd_down", T, d, f)]
    for name, M, N, K in shapes:
        x, w = torch.randn(M, K, device=dev, dtype=bf), torch.randn(N, K, device=dev, dtype=bf)
        out = torch.empty(M, N, device=dev, dtype=bf)
        us = t.run(lambda: G.gemm(x, w, out=out), a.iters)
        _emit("gemm", {"kind": name, "M": M, "N": N, "K": K}, us, flops=2.0 * M * N * K)
    # dgrad: dx = dy @ w, wgrad: dw = dy^T @ x with the squared-norm epilogue
    dy, w = torch.randn(T, 2 * f, device=dev, dtype=bf), torch.randn(2 * f, d, device=dev, dtype=bf)
    dx = torch.empty(T, d, device=dev, dtype=bf)
    us = t.run(lambda: G.gemm(dy, w, b_mn=True, out=dx), a.iters)
    _emit("gemm", {"kind": "dgrad_gate_up", "M": T, "N": d, "K": 2 * f}, us, flops=2.0 * T * d * 2 * f)
    x = torch.randn(T, d, device=dev, dtype=bf)
    dw = torch.empty(2 * f, d, device=dev, dtype=bf)
    ss = torch.zeros(1, dtype=torch.float64, device=dev)
    us = t.run(lambda: G.linear_wgrad(dy, x, out=dw, sumsq=ss), a.iters)
    _emit("gemm", {"kind": "wgrad_gate_up_sumsq", "M": 2 * f, "N": d, "K": T}, us, flops=2.0 * T * d * 2 * f)
    # down projection's input gradient: plain product + separate SwiGLU backward against the fused epilogue
    from opake_b200.ops import kernels as K
    dyd, wd = torch.randn(T, d, device=dev, dtype=bf), torch.randn(d, f, device=dev, dtype=bf) * 0.05
    gu, dgu = torch.randn(T, 2 * f, device=dev, dtype=bf), torch.empty(T, 2 * f, device=dev, dtype=bf)
    dact = torch.empty(T, f, device=dev, dtype=bf)

    def unfused():
        G.gemm(dyd, wd, b_mn=True, out=dact)
        K.swiglu_bwd(dact, gu, out=dgu)

    us = t.run(unfused, a.iters)
    _emit("gemm", {"kind": "dgrad_down_then_swiglu_bwd", "M": T, "N": f, "K": d}, us, flops=2.0 * T * d * f)
    us = t.run(lambda: G.swiglu_dgrad(dyd, wd, gu, out=dgu), a.iters)
    _emit("gemm", {"kind": "dgrad_down_swiglu_bwd_epilogue", "M": T, "N": f, "K": d}, us, flops=2.0 * T * d * f)


def case_attention(t: _Timer, a) -> None:
    from opake_b200.ops.flash import flash_bwd, flash_fwd
    dev = t.device
    T, H, KV, hd = (1024, 16, 4, 128) if a.small else (2048, 32, 8, 128)
    qkv = (torch.randn(T, (H + 2 * KV) * hd, device=dev) * 0.5).to(torch.bfloat16)
    dout = (torch.randn(T, H * hd, device=dev) * 0.5).to(torch.bfloat16)
    dqkv = torch.empty_like(qkv)
    out, lse = flash_fwd(qkv, H, KV, hd)
    causal_flops = 2.0 * 2 * H * hd * T * T / 2
    us = t.run(lambda: flash_fwd(qkv, H, KV, hd), a.iters)
    _emit("attention", {"kind": "forward", "T": T, "H": H, "KV": KV, "hd": hd}, us, flops=causal_flops)
    us = t.run(lambda: flash_bwd(dout, qkv, out, lse, H, KV, hd, dqkv), a.iters)
    _emit("attention", {"kind": "backward", "T": T, "H": H, "KV": KV, "hd": hd}, us, flops=2.5 * causal_flops)


def case_dp_step(t: _Timer, a) -> None:
    from opake_b200.ops import kernels as K
    dev = t.device
    n = (64 if a.small else 1024) << 20
    acc = torch.randn(n, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    p = torch.zeros(n, device=dev, dtype=torch.bfloat16)

    def step():
        K.dp_step(grad_src=[acc.data_ptr()], shard_begin=0, shard_len=n, inv_batch=1 / 256, sigma=1e-3, seed=1, step=0, m=m, v=v,
                  master=None, param_dst=[p.data_ptr()], param_src=p, lr=1e-4, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01,
                  bc1=0.1, bc2=0.001, phi_hat=1e-9, zero_grad=False, blt_state=None, blt_decay=None, blt_scale=None, sgd_mode=False,
                  device=dev)

    us = t.run(step, a.iters)
    _emit("dp_step", {"elements": n}, us, bytes_=n * (4 + 4 + 4 + 4 + 4 + 2 + 2))   # read g,m,v,p; write m,v,p


def case_clip_accumulate(t: _Timer, a) -> None:
    from opake_b200.ops import kernels as K
    dev = t.device
    n = (64 if a.small else 1024) << 20
    g = torch.randn(n, device=dev).to(torch.bfloat16)
    acc = torch.zeros(n, device=dev)
    scale = torch.full((1,), 0.37, device=dev)
    us = t.run(lambda: K.clip_accumulate(g, scale, acc), a.iters)
    _emit("clip_accumulate", {"elements": n}, us, bytes_=n * (2 + 4 + 4))


def case_rmsnorm(t: _Timer, a) -> None:
    from opake_b200.ops import kernels as K
    dev = t.device
    T, D = (8192, 4096) if a.small else (32768, 4096)
    x = torch.randn(T, D, device=dev).to(torch.bfloat16)
    w = torch.ones(D, device=dev, dtype=torch.bfloat16)
    y, rstd = K.rmsnorm_fwd(x, w)
    us = t.run(lambda: K.rmsnorm_fwd(x, w, out=y), a.iters)
    _emit("rmsnorm", {"kind": "forward", "T": T, "D": D}, us, bytes_=T * D * 4)
    dw = torch.zeros(D, device=dev)
    dx = torch.empty_like(x)
    us = t.run(lambda: K.rmsnorm_bwd(y, x, w, rstd, dw=dw, out=dx), a.iters)
    _emit("rmsnorm", {"kind": "backward", "T": T, "D": D}, us, bytes_=T * D * 6)


def case_lce(t: _Timer, a) -> None:
    from opake_b200.ops import gemm as G, kernels as K
    dev = t.device
    T, D, V = (1024, 2048, 32000) if a.small else (2048, 4096, 128256)
    h = (torch.randn(T, D, device=dev) * 0.3).to(torch.bfloat16)
    W = (torch.randn(V, D, device=dev) * 0.05).to(torch.bfloat16)
    lab = torch.randint(0, V, (T,), device=dev, dtype=torch.int32)
    tiles = G.lce_tiles(V)
    pmax, psum = torch.empty(T, tiles, device=dev), torch.empty(T, tiles, device=dev)
    tgt = torch.empty(T, device=dev)

    def fwd():
        G.gemm(h, W, epilogue=G.EPI_LCE_FWD, labels=lab, pmax=pmax, psum=psum, tgt=tgt)
        return K.lce_finalize(pmax, psum, tgt, lab)

    us = t.run(fwd, a.iters)
    _emit("lce", {"kind": "forward", "T": T, "D": D, "V": V}, us, flops=2.0 * T * D * V)


def case_clip_sum(t: _Timer, a) -> None:
    from opake_b200.ops.clip_sum import fused_clip_sum
    dev = t.device
    B, n = (8, 16 << 20) if a.small else (16, 64 << 20)
    leaves = [torch.randn(B, n, device=dev).to(torch.bfloat16)]
    us = t.run(lambda: fused_clip_sum(leaves, 1.0), a.iters)
    _emit("clip_sum", {"B": B, "elements": n}, us, bytes_=2.0 * B * n * 2 + 4 * n)


def case_moe(t: _Timer, a) -> None:
    """One mixture-of-experts layer on one GPU (OLMoE shape): router product, top-k routing and row plan, gather by
    expert, grouped gate/up GEMM with the SwiGLU epilogue, grouped down GEMM, weighted combine with the residual."""
    from opake_b200.ops import gemm as G, kernels as K
    dev = t.device
    T, d, E, k, I = (1024, 1024, 32, 4, 512) if a.small else (2048, 2048, 64, 8, 1024)
    x = (torch.randn(T, d, device=dev) * 0.5).to(torch.bfloat16)
    router = (torch.randn(E, d, device=dev) * 0.05).to(torch.bfloat16)
    wgu = (torch.randn(E, 2 * I, d, device=dev) * 0.03).to(torch.bfloat16)
    wd = (torch.randn(E, d, I, device=dev) * 0.03).to(torch.bfloat16)
    plan = K.MoePlan(T, E, k, dev)
    e = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)  # noqa: E731
    rl, xs, gu, act, ye, out = e(T, E), e(plan.R, d), e(plan.R, 2 * I), e(plan.R, I), e(plan.R, d), e(T, d)

    def route():
        G.gemm(x, router, out=rl)
        K.moe_route(rl, plan, False)

    def experts():
        K.moe_gather(x, plan, xs)
        G.gemm(xs, wgu, out=gu, epilogue=G.EPI_SWIGLU, act=act, tile_group=plan.tile_group)
        G.gemm(act, wd, out=ye, tile_group=plan.tile_group)
        K.moe_combine(ye, plan, out, wts=plan.wts, residual=x)

    route()
    us_r = t.run(route, a.iters)
    _emit("moe", {"kind": "router + top-k + row plan", "T": T, "E": E, "k": k}, us_r, flops=2.0 * T * d * E)
    us_e = t.run(experts, a.iters)
    # useful work: every token visits k experts, each 3 * I * d multiply-adds (gate, up, down)
    _emit("moe", {"kind": "gather + grouped GEMMs (SwiGLU epilogue) + combine", "T": T, "d": d, "E": E, "k": k, "ffn": I, "rows": plan.R},
          us_e, flops=2.0 * T * k * 3 * I * d)


CASES = {"moe": case_moe, "gemm": case_gemm, "attention": case_attention, "dp_step": case_dp_step, "clip_accumulate": case_clip_accumulate,
         "rmsnorm": case_rmsnorm, "lce": case_lce, "clip_sum": case_clip_sum}


def main(argv=None) -> int:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("case", choices=sorted(CASES) + ["all"])
    p.add_argument("--iters", type=int, default=10)
    p.add_argument("--small", action="store_true")
    p.add_argument("--once", action="store_true")
    a = p.parse_args(argv)
    if not torch.cuda.is_available():
        print("a CUDA device is required", file=sys.stderr)
        return 2
    if a.once:
        a.iters = 1
    dev = torch.device("cuda", torch.cuda.current_device())
    timer = _Timer(dev)
    for name in (sorted(CASES) if a.case == "all" else [a.case]):
        CASES[name](timer, a)
    from opake_b200.ops._lib import raise_if_device_error
    raise_if_device_error(dev)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
