"""Sharded DP-SGD / DP-FTRL training engine for the native decoder runtimes.

Per optimizer step (logical batch of B sequences, B / W per rank):

1. every rank runs its examples one at a time through ``DecoderRuntime.example_grad`` (tensor-core GEMMs with the
   per-example norm reduced in the weight-gradient epilogues), clips and adds them into its fp32 sum ``acc``;
2. one fused kernel per rank (``opk_dp_step``) then *reduce-scatters* the sums by reading its shard of every peer's
   ``acc`` over NVLink, normalises by B, adds Philox Gaussian noise indexed by the global element offset (each
   element is owned by exactly one rank, so noise is added exactly once), optionally passes the noise through the
   buffered-linear-Toeplitz correlation state (DP-FTRL), applies DP-AdamW with noise bias correction on the rank's
   fp32 moment shard, and *all-gathers* by storing the updated bf16 parameters into every peer's replica.

Persistent state per rank: bf16 parameter replica (P*2 B), fp32 ``acc`` (P*4 B), bf16 per-example gradient ``G``
(P*2 B), and 1/W of the fp32 moments (and master weights when enabled). The reference keeps replicated parameters and
optimizer state and all-reduces every gradient leaf separately (packages/opake-engine/src/opake/api/engine/distributed/
gradients.py:150-200) with CPU-generated noise (packages/opake-dpsgd/src/opake/api/dpsgd/noise/_gaussian.py:188-204).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..models.config import DecoderConfig
from ..models.decoder import DecoderRuntime, init_params_
from ..models.flat import build_layout
from ..ops import kernels as K
from . import comm

_bf16 = torch.bfloat16


@dataclass
class EngineConfig:
    clip_norm: float = 1.0
    noise_multiplier: float = 1.0
    logical_batch: int = 256           # normalize_by: the global (expected) batch size
    lr: float = 3e-4
    betas: tuple[float, float] = (0.9, 0.999)
    eps: float = 1e-8
    weight_decay: float = 0.01
    noise_bias_correction: bool = True  # AdamW-BC
    master_weights: bool = False
    optimizer: str = "adamw"            # "adamw" | "sgd"
    auto_clip: bool = False             # AUTO-S: R / (norm + gamma)
    auto_gamma: float = 0.01
    seed: int = 0
    use_cuda_graph: bool = True
    attn_impl: str = "auto"
    # DP-FTRL: buffered linear Toeplitz correlated noise (decay, scale per buffer); empty = independent noise
    blt_decay: tuple[float, ...] = ()
    blt_scale: tuple[float, ...] = ()
    noise_stream_tag: str = "opake.dpsgd.gaussian"
    accumulate_group: int = 0           # whole-model gradient buffers per accumulation pass; 0 = as many as fit (2..6)


class ShardedDPEngine:
    def __init__(self, model_cfg: DecoderConfig, cfg: EngineConfig, device: torch.device, *, init_seed: int = 0):
        self.model_cfg, self.cfg, self.device = model_cfg, cfg, device
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.layout = build_layout(model_cfg, shard_multiple=self.world)
        total = self.layout.total
        self.shard_len = total // self.world
        self.shard_begin = self.rank * self.shard_len
        # peer-addressable buffers
        self.params_pb = comm.alloc_peer_buffer(total, _bf16, device)
        self.acc_pb = comm.alloc_peer_buffer(total, torch.float32, device)
        self.params, self.acc = self.params_pb.local, self.acc_pb.local
        init_params_(model_cfg, self.params, self.layout, seed=init_seed)  # same seed on every rank -> same replica
        self.acc.zero_()
        self.m = torch.zeros(self.shard_len, dtype=torch.float32, device=device)
        self.v = torch.zeros(self.shard_len, dtype=torch.float32, device=device)
        self.master = None
        if cfg.master_weights:
            self.master = self.params[self.shard_begin : self.shard_begin + self.shard_len].float()
        self.blt_state = self.blt_decay = self.blt_scale = None
        if cfg.blt_decay:
            nb = len(cfg.blt_decay)
            self.blt_state = torch.zeros(nb, self.shard_len, dtype=torch.float32, device=device)
            self.blt_decay = torch.tensor(cfg.blt_decay, dtype=torch.float32, device=device)
            self.blt_scale = torch.tensor(cfg.blt_scale, dtype=torch.float32, device=device)
        if cfg.accumulate_group and not 2 <= int(cfg.accumulate_group) <= 8:
            raise ValueError(f"accumulate_group must be 0 (automatic) or between 2 and 8, got {cfg.accumulate_group}")
        self.group = int(cfg.accumulate_group) or self._pick_group_size()
        self.runtime = DecoderRuntime(model_cfg, self.params, layout=self.layout, attn_impl=cfg.attn_impl, n_slots=self.group)
        self._side = torch.cuda.Stream(device=device)
        self._warm: dict[int, bool] = {}
        self.step_count = 0
        self.phi = 0.0
        from ..engine.random import fold_in, key

        self._noise_key = key(cfg.seed)
        self._fold_in = fold_in
        self._graphs: dict[int, tuple] = {}
        self._losses = None
        self.graph_kernel_launches = 0   # native launches replayed through CUDA graphs (not seen by the ctypes counter)

    def _pick_group_size(self) -> int:
        """How many whole-model bf16 gradient buffers to keep: the clipped accumulation reads and writes the fp32
        sums once per GROUP of examples (2 + 8 / group bytes per parameter and example), so more buffers mean less HBM
        traffic. Sharding the optimizer state over more ranks frees the memory for them.
        ``EngineConfig.accumulate_group`` overrides the automatic choice."""
        if self.device.type != "cuda":
            return 2
        free, _ = torch.cuda.mem_get_info(self.device)
        g_bytes = 2 * self.layout.dense_total
        # Reserve for activations, workspaces, CUDA-graph pools and allocator slack. Measured on one 178 GB device with
        # an 8B model: 142 GB in use with a group of 2, 14 GB more per additional buffer; 20 GB of reserve leave at
        # least 21 GB free in every 1 / 2 / 4 / 8-GPU configuration. Groups above 6 are not used automatically.
        reserve = 20 << 30 if g_bytes > (4 << 30) else 4 * g_bytes + (2 << 30)
        cap = 6 if g_bytes > (4 << 30) else 8
        return int(max(2, min(cap, (free - reserve) // max(g_bytes, 1))))

    # ------------------------------------------------------------------ one example
    def _example_body(self, ws, slot: int, drain_prev: bool) -> None:
        """Gradient of the example staged in slot ``slot``; meanwhile (side stream) the clipped accumulation of the
        previous example, which sits in the other slot. HBM-bound accumulation and tensor-core-bound GEMMs share
        the SMs, so the accumulation is hidden."""
        rt, cfg = self.runtime, self.cfg
        main = torch.cuda.current_stream(self.device)
        # examples cycle through the gradient buffers; when the last buffer of the group is full, all of them are
        # clipped and added in a single pass over the fp32 sums (2 + 8 / group bytes of HBM traffic per parameter
        # and example instead of 10)
        # The pass itself is deferred to the start of the NEXT group's first example and runs on the side stream
        # under that example's forward GEMMs (HBM-bound next to tensor-core-bound work); the example waits for it
        # right before its first weight-gradient GEMM, the first kernel that overwrites a gradient buffer.
        hook = None
        if drain_prev and slot == 0:
            self._side.wait_stream(main)
            with torch.cuda.stream(self._side):
                rt.accumulate_group(self.acc, ws, self.group, toks=self._group_toks(ws, self.group))
            hook = lambda: main.wait_stream(self._side)
        st = rt.example_grad(ws["toks"][slot], ws["labels"], ws=ws, slot=slot, before_wgrad=hook)
        rt.clip_factor(cfg.clip_norm, auto=cfg.auto_clip, gamma=cfg.auto_gamma, slot=slot)
        ws["loss_sum"].add_(st.loss.reshape(1))
        if slot == 0:
            ws["tok_keep"].copy_(ws["toks"][0])      # slot 0's tokens are replaced before its deferred pass runs

    @staticmethod
    def _group_toks(ws, n: int):
        return [ws["tok_keep"], *ws["toks"][1:n]]

    def _run_example(self, tok_host: torch.Tensor, labels_host: torch.Tensor, index: int) -> None:
        T = tok_host.numel()
        ws = self.runtime.workspace(T)
        slot = index % self.group
        drain = index > 0
        ws["toks"][slot].copy_(tok_host, non_blocking=True)
        ws["labels"].copy_(labels_host, non_blocking=True)
        if not self.cfg.use_cuda_graph:
            self._example_body(ws, slot, drain)
            return
        key = (T, slot, drain)
        entry = self._graphs.get(key)
        if entry is None:
            from ..ops import _lib

            if not self._warm.get(T):
                # eager warm-up (lazy workspaces, library autotuning) on a side stream, state restored afterwards
                saved = (ws["loss_sum"].clone(), self.acc.clone() if self.acc.numel() < (1 << 28) else None)
                s = torch.cuda.Stream(device=self.device)
                s.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(s):
                    self._example_body(ws, slot, False)
                torch.cuda.current_stream(self.device).wait_stream(s)
                torch.cuda.synchronize(self.device)
                ws["loss_sum"].copy_(saved[0])
                self.runtime.clip_count.zero_()
                self._warm[T] = True
            g = torch.cuda.CUDAGraph()
            before = _lib.LAUNCHES[0]
            with torch.cuda.graph(g):
                self._example_body(ws, slot, drain)
            entry = (g, _lib.LAUNCHES[0] - before)
            self._graphs[key] = entry
            # capture does not execute: fall through to the first replay
        entry[0].replay()
        self.graph_kernel_launches += entry[1]

    # ------------------------------------------------------------------ optimizer step
    def _noise_sigma(self) -> float:
        return self.cfg.noise_multiplier * self.cfg.clip_norm / self.cfg.logical_batch

    def step(self, tokens: torch.Tensor, labels: torch.Tensor) -> torch.Tensor:
        """One DP optimizer step on this rank's slice of the logical batch.

        ``tokens`` / ``labels``: pinned host int32 ``[B_local, T]`` (labels shifted, negative = ignored).
        Returns the device tensor holding the sum of this rank's example losses (read it with ``.item()``).
        """
        cfg = self.cfg
        B_local = tokens.shape[0]
        ws = self.runtime.workspace(tokens.shape[1])
        if "loss_sum" not in ws:
            ws["loss_sum"] = torch.zeros(1, dtype=torch.float32, device=self.device)
        if "tok_keep" not in ws:
            ws["tok_keep"] = torch.zeros_like(ws["toks"][0])
        ws["loss_sum"].zero_()
        for i in range(B_local):
            self._run_example(tokens[i], labels[i], i)
        # the last group (complete or not) has not been added yet: every earlier one was added at the start of the
        # example that followed it
        n_last = B_local % self.group or min(self.group, B_local)
        if n_last:
            self.runtime.accumulate_group(self.acc, ws, n_last, toks=self._group_toks(ws, n_last))
        loss_sum = ws["loss_sum"].clone()
        self.apply_update()
        return loss_sum

    def apply_update(self) -> None:
        cfg = self.cfg
        t = self.step_count + 1
        b1, b2 = cfg.betas
        sigma = self._noise_sigma()
        step_key = self._fold_in(self._noise_key, cfg.noise_stream_tag, self.step_count)
        phi_hat = 0.0
        if cfg.noise_bias_correction and cfg.optimizer == "adamw":
            self.phi = b2 * self.phi + (1.0 - b2) * sigma * sigma
            phi_hat = self.phi / (1.0 - b2**t)
        if self.world > 1:
            self.acc_pb.barrier()       # every rank finished accumulating before anyone reads peers' sums
        K.dp_step(
            grad_src=self._rotate(self.acc_pb.ptrs), shard_begin=self.shard_begin, shard_len=self.shard_len,
            inv_batch=1.0 / cfg.logical_batch, sigma=sigma, seed=step_key.seed, step=self.step_count,
            m=self.m, v=self.v, master=self.master, param_dst=self._rotate(self.params_pb.ptrs), param_src=self.params,
            lr=cfg.lr, beta1=b1, beta2=b2, eps=cfg.eps, weight_decay=cfg.weight_decay, bc1=1.0 - b1**t,
            bc2=1.0 - b2**t, phi_hat=phi_hat, zero_grad=False, blt_state=self.blt_state, blt_decay=self.blt_decay,
            blt_scale=self.blt_scale, sgd_mode=(cfg.optimizer == "sgd"), device=self.device)
        if self.world > 1:
            self.params_pb.barrier()    # all shards of the new parameters have landed everywhere
        self.acc.zero_()
        self.step_count += 1

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> dict:
        """This rank's shard of the training state (parameters are replicated, so rank 0's copy suffices for them)."""
        out = {"step_count": self.step_count, "phi": float(self.phi), "shard_begin": self.shard_begin,
               "shard_len": self.shard_len, "world": self.world, "m": self.m.cpu(), "v": self.v.cpu(),
               "master": None if self.master is None else self.master.cpu(),
               "blt_state": None if self.blt_state is None else self.blt_state.cpu(),
               "noise_key": {"seed": self._noise_key.seed, "impl": self._noise_key.impl}}
        if self.rank == 0:
            out["params"] = self.params.cpu()
        return out

    def load_state_dict(self, sd: dict, params: torch.Tensor | None = None) -> None:
        if sd["world"] != self.world or sd["shard_len"] != self.shard_len:
            raise ValueError(f"engine checkpoint was written with world size {sd['world']} (shard {sd['shard_len']}); "
                             f"this run has world size {self.world} (shard {self.shard_len})")
        self.step_count, self.phi = int(sd["step_count"]), float(sd["phi"])
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        if self.master is not None and sd.get("master") is not None:
            self.master.copy_(sd["master"])
        if self.blt_state is not None and sd.get("blt_state") is not None:
            self.blt_state.copy_(sd["blt_state"])
        p = sd.get("params") if params is None else params
        if p is not None:
            self.params.copy_(p)

    def _rotate(self, ptrs: list[int]) -> list[int]:
        """This rank's buffer first, then the peers starting at rank+1 (spreads NVLink traffic across peers)."""
        r = self.rank
        return [ptrs[(r + i) % len(ptrs)] for i in range(len(ptrs))]
