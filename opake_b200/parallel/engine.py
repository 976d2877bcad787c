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
from ..engine.profiling import nvtx_range
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
    # DP-FTRL with a banded Toeplitz strategy (band-MF, banded square root): first column of C; () = not used
    toeplitz_coef: tuple[float, ...] = ()
    # Full sharding (both need more than one rank to change anything):
    #   shard_params  every parameter tensor has one owner; the optimizer step writes only the owner's copy and the
    #                 other ranks fetch it inside the first forward GEMM that consumes it (all-gather fused into the GEMM)
    #   shard_sums    the fp32 clipped-gradient sums are sharded like the optimizer state; each accumulation group is
    #                 reduce-scattered to the owners with reductions over NVLink while the next group's forward runs
    shard_params: bool = False
    shard_sums: bool = False
    # Expert parallelism for mixture-of-experts models on more than one rank: every rank keeps n_experts / world experts
    # of every layer (parameters, sums and moments), tokens travel to the owners; needs the sequence length up front
    expert_parallel: bool = False
    seq_len: int = 0
    # "peer": the fused step reads / writes the other ranks' buffers itself (NVLink loads and stores inside the kernel).
    # "nccl": the same step with library collectives around a local kernel (reduce_scatter_tensor before, in-place
    # all_gather_into_tensor after): the baseline and fallback implementation of the same interface.
    comm_backend: str = "peer"
    # debugging aid: gradient slots and workspaces sit between guard bands that are verified after every step
    debug_canaries: bool = False


class ShardedDPEngine:
    def __init__(self, model_cfg: DecoderConfig, cfg: EngineConfig, device: torch.device, *, init_seed: int = 0):
        self.model_cfg, self.cfg, self.device = model_cfg, cfg, device
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        self.expert_parallel = bool(cfg.expert_parallel) and bool(model_cfg.n_experts) and self.world > 1
        if self.expert_parallel and cfg.seq_len <= 0:
            raise ValueError("expert parallelism sizes its token buffers at start-up: set EngineConfig.seq_len")
        self.layout = build_layout(model_cfg, shard_multiple=self.world, skip_experts=self.expert_parallel)
        total = self.layout.total
        self.shard_params = bool(cfg.shard_params) and self.world > 1
        self.shard_sums = bool(cfg.shard_sums) and self.world > 1
        if self.shard_params or self.shard_sums:
            self.bounds = self.layout.shard_bounds(self.world)      # every tensor has exactly one owner
        else:
            self.bounds = [r * (total // self.world) for r in range(self.world)] + [total]
        self.shard_begin = self.bounds[self.rank]
        self.shard_len = self.bounds[self.rank + 1] - self.shard_begin
        # peer-addressable buffers
        self.params_pb = comm.alloc_peer_buffer(total, _bf16, device)
        self.params = self.params_pb.local
        if self.shard_sums:
            longest = max(self.bounds[r + 1] - self.bounds[r] for r in range(self.world))
            self.acc_pb = comm.alloc_peer_buffer(max(longest, 8), torch.float32, device)    # this rank's shard only
        else:
            self.acc_pb = comm.alloc_peer_buffer(total, torch.float32, device)
        self.acc = self.acc_pb.local
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
        self.toep_state = self.toep_coef = None
        self.toep_pos = 0
        if cfg.toeplitz_coef:
            if cfg.blt_decay:
                raise ValueError("choose one correlated-noise strategy: buffered linear Toeplitz or banded Toeplitz")
            if cfg.toeplitz_coef[0] == 0:
                raise ValueError("the leading Toeplitz coefficient must be non-zero")
            self.toep_coef = torch.tensor(cfg.toeplitz_coef, dtype=torch.float32, device=device)
            nlag = len(cfg.toeplitz_coef) - 1
            if nlag:
                self.toep_state = torch.zeros(nlag, self.shard_len, dtype=torch.float32, device=device)
        if cfg.comm_backend not in ("peer", "nccl"):
            raise ValueError(f"comm_backend must be 'peer' or 'nccl', got {cfg.comm_backend!r}")
        self.nccl_step = cfg.comm_backend == "nccl" and self.world > 1
        if self.nccl_step and (self.shard_params or self.shard_sums):
            raise ValueError("the NCCL baseline step works on replicated parameters and sums (shard_params / shard_sums off)")
        self._rs_out = torch.empty(self.shard_len, dtype=torch.float32, device=device) if self.nccl_step else None
        self._stale = False      # shard_params: the replica's remote parts are older than their owners' copies
        self._refresh: dict[int, tuple] = {}
        if cfg.accumulate_group and not 2 <= int(cfg.accumulate_group) <= 8:
            raise ValueError(f"accumulate_group must be 0 (automatic) or between 2 and 8, got {cfg.accumulate_group}")
        self.group = int(cfg.accumulate_group) or self._pick_group_size()
        self.ep = None
        if self.expert_parallel:
            from .ep_runtime import ExpertParallelRuntime

            views = self.layout.views(self.params)
            routers = [views[f"layers.{i}.router"] for i in range(model_cfg.n_layers)]
            self.ep = ExpertParallelRuntime(model_cfg, routers, cfg.seq_len, device, init_seed=init_seed)
        self.canaries = None
        if cfg.debug_canaries:
            from ..utils.canary import CanaryPool

            self.canaries = CanaryPool(device)
        self.runtime = DecoderRuntime(model_cfg, self.params, layout=self.layout, attn_impl=cfg.attn_impl, n_slots=self.group,
                                      ep=self.ep, canaries=self.canaries)
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
        if self.world > 1:
            # every rank's buffers are initialised before any peer reads or adds to them
            torch.cuda.synchronize(device)
            dist.barrier()

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
        # with sharded sums every accumulation pass crosses NVLink, so a larger group pays directly: up to 8 there
        cap = 8 if (g_bytes <= (4 << 30) or getattr(self, "shard_sums", False)) else 6
        return int(max(2, min(cap, (free - reserve) // max(g_bytes, 1))))

    # ------------------------------------------------------------------ one example
    # ------------------------------------------------------------------ sharding helpers
    def _refresh_plan(self, T: int) -> tuple:
        """What a refresh of the replica fetches from other ranks, for sequences of ``T`` tokens: ``fetch`` maps the
        weights whose first forward GEMM can pull them itself (staged two-CTA kernel) to the owner's copy; ``copies``
        lists the remaining remote ranges (norm weights, biases, embeddings, LM head) as (element offset, elements,
        owner), merged into maximal runs, for the plain peer-copy kernel."""
        plan = self._refresh.get(T)
        if plan is not None:
            return plan
        fetch, copies = {}, []
        act = self.model_cfg.act
        for sl in self.layout.slots:
            owner = self.layout.owner_of(sl.name, self.bounds)
            if owner == self.rank:
                continue
            if DecoderRuntime.stageable(sl.name, sl.shape, T, act) and not self.model_cfg.n_experts:
                fetch[sl.name] = self.params_pb.peer_view(owner, sl.shape, offset=sl.offset)
                continue
            n = (sl.numel + 127) // 128 * 128
            if copies and copies[-1][2] == owner and copies[-1][0] + copies[-1][1] == sl.offset:
                copies[-1] = (copies[-1][0], copies[-1][1] + n, owner)
            else:
                copies.append((sl.offset, n, owner))
        plan = (fetch, copies)
        self._refresh[T] = plan
        return plan

    def _accumulate(self, ws, n: int, toks) -> None:
        """Adds the clipped gradients held in slots ``0 .. n-1`` to the fp32 sums (local pass, or reductions into the
        owners' shards when the sums are sharded)."""
        if not self.shard_sums:
            self.runtime.accumulate_group(self.acc, ws, n, toks=toks)
            return
        emb_acc = None
        if not self.model_cfg.tie_embeddings:
            emb = self.layout.slot("embed")
            owner = self.layout.owner_of("embed", self.bounds)
            emb_acc = self.acc_pb.peer_view(owner, emb.shape, offset=emb.offset - self.bounds[owner])
        self.runtime.accumulate_group_sharded(self.acc_pb.ptrs, self.bounds, self.rank, ws, n, emb_acc=emb_acc, toks=toks)

    def _example_body(self, ws, slot: int, drain_prev: bool, refresh: bool = False) -> None:
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
                self._accumulate(ws, self.group, self._group_toks(ws, self.group))
            hook = lambda: main.wait_stream(self._side)
        if refresh:
            # first example after an optimizer step with sharded parameters: small tensors come over with the copy
            # kernel, the layer matrices inside the forward GEMMs that consume them
            fetch, copies = self._refresh_plan(ws["toks"][slot].numel())
            for off, n, owner in copies:
                K.copy_bytes(self.params.data_ptr() + 2 * off, self.params_pb.ptrs[owner] + 2 * off, 2 * n, self.device)
            rt._fetch = fetch
        if self.ep is not None:
            self.ep.begin_example()
        try:
            st = rt.example_grad(ws["toks"][slot], ws["labels"], ws=ws, slot=slot, before_wgrad=hook)
        finally:
            rt._fetch = None
        if self.ep is not None:
            # the example's squared norm has parts on every rank that owns experts: combine them, derive every
            # example's clip factor, and form the clipped expert-gradient sums (pass 2) while the rows are still there
            scales = self.ep.clip_factors(rt.sumsqs[slot], cfg.clip_norm, auto=cfg.auto_clip, gamma=cfg.auto_gamma,
                                          n_leaves=rt._n_leaves + 2 * self.model_cfg.n_layers,
                                          widest_leaf=max(rt._widest, self.ep.n_wgu), counters=rt.clip_count)
            rt.scales[slot].copy_(scales[self.rank : self.rank + 1])
            self.ep.accumulate_clipped()
            self.ep.end_example()
        else:
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
        refresh = index == 0 and self._stale
        if refresh:
            self._stale = False
        ws["toks"][slot].copy_(tok_host, non_blocking=True)
        ws["labels"].copy_(labels_host, non_blocking=True)
        if not self.cfg.use_cuda_graph:
            self._example_body(ws, slot, drain, refresh)
            return
        key = (T, slot, drain, refresh)
        entry = self._graphs.get(key)
        if entry is None:
            from ..ops import _lib

            if not self._warm.get((T, refresh)):
                # eager warm-up (lazy workspaces, library autotuning) on a side stream, state restored afterwards
                saved = (ws["loss_sum"].clone(), self.acc.clone() if self.acc.numel() < (1 << 28) else None)
                s = torch.cuda.Stream(device=self.device)
                s.wait_stream(torch.cuda.current_stream(self.device))
                with torch.cuda.stream(s):
                    self._example_body(ws, slot, False, refresh)
                torch.cuda.current_stream(self.device).wait_stream(s)
                torch.cuda.synchronize(self.device)
                ws["loss_sum"].copy_(saved[0])
                self.runtime.clip_count.zero_()
                if self.ep is not None:
                    # warm-ups only ever happen on the first example of a step, where the expert sums are still zero
                    self.ep.acc.zero_()
                self._warm[(T, refresh)] = True
            g = torch.cuda.CUDAGraph()
            before = _lib.LAUNCHES[0]
            with torch.cuda.graph(g):
                self._example_body(ws, slot, drain, refresh)
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
        if self.ep is not None:
            if tokens.shape[1] != self.cfg.seq_len:
                raise ValueError(f"expert-parallel buffers were sized for sequences of {self.cfg.seq_len} tokens")
            # the exchange kernels wait for their peers with a bounded budget: start every step together
            torch.cuda.synchronize(self.device)
            dist.barrier()
        ws = self.runtime.workspace(tokens.shape[1])
        if "loss_sum" not in ws:
            ws["loss_sum"] = torch.zeros(1, dtype=torch.float32, device=self.device)
        if "tok_keep" not in ws:
            ws["tok_keep"] = torch.zeros_like(ws["toks"][0])
        ws["loss_sum"].zero_()
        with nvtx_range("opake::examples"):
            for i in range(B_local):
                self._run_example(tokens[i], labels[i], i)
        # the last group (complete or not) has not been added yet: every earlier one was added at the start of the
        # example that followed it
        n_last = B_local % self.group or min(self.group, B_local)
        if n_last:
            self._accumulate(ws, n_last, self._group_toks(ws, n_last))
        loss_sum = ws["loss_sum"].clone()
        with nvtx_range("opake::dp_step"):
            self.apply_update()
        if self.canaries is not None:
            self.canaries.assert_intact()       # synchronises; raises DeviceIntegrityError naming the damaged buffer
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
        if self.nccl_step:
            self._apply_update_nccl(sigma, step_key, phi_hat, t)
            return
        if self.world > 1:
            self.acc_pb.barrier()       # every rank finished accumulating before anyone reads (or owns) the sums
        if self.shard_sums:
            # the owner's shard already holds the sum over all ranks; addressed with global offsets like a full buffer
            grad_src = [self.acc.data_ptr() - 4 * self.shard_begin]
        else:
            grad_src = self._rotate(self.acc_pb.ptrs)
        # sharded parameters: only the owner's copy is written here, the other ranks fetch it in their next forward pass
        param_dst = [self.params.data_ptr()] if self.shard_params else self._rotate(self.params_pb.ptrs)
        K.dp_step(
            grad_src=grad_src, shard_begin=self.shard_begin, shard_len=self.shard_len,
            inv_batch=1.0 / cfg.logical_batch, sigma=sigma, seed=step_key.seed, step=self.step_count,
            m=self.m, v=self.v, master=self.master, param_dst=param_dst, param_src=self.params,
            lr=cfg.lr, beta1=b1, beta2=b2, eps=cfg.eps, weight_decay=cfg.weight_decay, bc1=1.0 - b1**t,
            bc2=1.0 - b2**t, phi_hat=phi_hat, zero_grad=self.shard_sums, blt_state=self.blt_state, blt_decay=self.blt_decay,
            blt_scale=self.blt_scale, toep_state=self.toep_state, toep_coef=self.toep_coef, toep_pos=self.toep_pos,
            sgd_mode=(cfg.optimizer == "sgd"), device=self.device)
        if self.ep is not None:
            self.ep.apply_update(noise_offset=self.layout.total, inv_batch=1.0 / cfg.logical_batch, sigma=sigma, seed=step_key.seed,
                                 step=self.step_count, lr=cfg.lr, beta1=b1, beta2=b2, eps=cfg.eps, weight_decay=cfg.weight_decay,
                                 bc1=1.0 - b1**t, bc2=1.0 - b2**t, phi_hat=phi_hat, sgd_mode=(cfg.optimizer == "sgd"))
        if self.toep_state is not None:
            self.toep_pos = (self.toep_pos - 1) % self.toep_state.shape[0]
        if self.world > 1:
            self.params_pb.barrier()    # the new parameters (and, sharded sums, the zeroed shards) are in place everywhere
        if not self.shard_sums:
            self.acc.zero_()
        if self.shard_params:
            self._stale = True
        self.step_count += 1

    def _apply_update_nccl(self, sigma: float, step_key, phi_hat: float, t: int) -> None:
        """The optimizer step on library collectives: NCCL reduce-scatter of the fp32 sums, the step kernel on local
        memory only, NCCL all-gather of the updated bf16 shards (in place: every rank's shard already sits at its
        offset of the replica)."""
        cfg = self.cfg
        b1, b2 = cfg.betas
        with nvtx_range("opake::dp_step/nccl"):
            dist.reduce_scatter_tensor(self._rs_out, self.acc[: self.shard_len * self.world], op=dist.ReduceOp.SUM)
            K.dp_step(
                grad_src=[self._rs_out.data_ptr() - 4 * self.shard_begin], shard_begin=self.shard_begin, shard_len=self.shard_len,
                inv_batch=1.0 / cfg.logical_batch, sigma=sigma, seed=step_key.seed, step=self.step_count,
                m=self.m, v=self.v, master=self.master, param_dst=[self.params.data_ptr()], param_src=self.params,
                lr=cfg.lr, beta1=b1, beta2=b2, eps=cfg.eps, weight_decay=cfg.weight_decay, bc1=1.0 - b1**t,
                bc2=1.0 - b2**t, phi_hat=phi_hat, zero_grad=False, blt_state=self.blt_state, blt_decay=self.blt_decay,
                blt_scale=self.blt_scale, toep_state=self.toep_state, toep_coef=self.toep_coef, toep_pos=self.toep_pos,
                sgd_mode=(cfg.optimizer == "sgd"), device=self.device)
            if self.toep_state is not None:
                self.toep_pos = (self.toep_pos - 1) % self.toep_state.shape[0]
            mine = self.params[self.shard_begin : self.shard_begin + self.shard_len]
            dist.all_gather_into_tensor(self.params[: self.shard_len * self.world], mine)
        self.acc.zero_()
        self.step_count += 1

    def gather_params(self) -> None:
        """Brings this rank's replica up to date outside a training step (evaluation, checkpointing): every remote
        range is copied from its owner with the peer-copy kernel. No-op unless the parameters are sharded and stale."""
        if not self._stale:
            return
        for r in range(self.world):
            if r == self.rank or self.bounds[r + 1] == self.bounds[r]:
                continue
            off, n = self.bounds[r], self.bounds[r + 1] - self.bounds[r]
            K.copy_bytes(self.params.data_ptr() + 2 * off, self.params_pb.ptrs[r] + 2 * off, 2 * n, self.device)
        self._stale = False

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self) -> dict:
        """This rank's shard of the training state (parameters are replicated, so rank 0's copy suffices for them)."""
        out = {"step_count": self.step_count, "phi": float(self.phi), "shard_begin": self.shard_begin,
               "shard_len": self.shard_len, "world": self.world, "m": self.m.cpu(), "v": self.v.cpu(),
               "master": None if self.master is None else self.master.cpu(),
               "blt_state": None if self.blt_state is None else self.blt_state.cpu(),
               "toep_state": None if self.toep_state is None else self.toep_state.cpu(), "toep_pos": self.toep_pos,
               "bounds": list(self.bounds),
               "noise_key": {"seed": self._noise_key.seed, "impl": self._noise_key.impl}}
        if self.rank == 0:
            self.gather_params()
            out["params"] = self.params.cpu()
        if self.ep is not None:
            out["experts"] = self.ep.state_dict()
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
        if self.toep_state is not None and sd.get("toep_state") is not None:
            self.toep_state.copy_(sd["toep_state"])
            self.toep_pos = int(sd.get("toep_pos", 0))
        p = sd.get("params") if params is None else params
        if p is not None:
            self.params.copy_(p)
        if self.ep is not None and sd.get("experts") is not None:
            self.ep.load_state_dict(sd["experts"])

    @staticmethod
    def consolidate(shards: list[dict]) -> dict:
        """One full-size training state from the per-rank ``state_dict()`` results of a run (any order): parameters from
        the rank that stored them, the optimizer moments (and master weights, correlated-noise state) concatenated in
        flat-parameter order. This is the layout a one-rank engine of the same model loads, and the one to convert
        into framework-neutral checkpoints."""
        if not shards:
            raise ValueError("no shards")
        world = int(shards[0]["world"])
        by_begin = sorted(shards, key=lambda sd: (int(sd["shard_begin"]), int(sd["shard_len"])))
        if len(by_begin) != world or any(int(sd["world"]) != world for sd in by_begin):
            raise ValueError(f"expected the {world} shards of one run")
        cursor = 0
        for sd in by_begin:
            if int(sd["shard_begin"]) != cursor:
                raise ValueError("shards do not tile the parameter vector (missing or duplicated rank)")
            cursor += int(sd["shard_len"])
        params = next((sd["params"] for sd in by_begin if sd.get("params") is not None), None)
        if params is None:
            raise ValueError("no shard carries the parameters (rank 0's file is missing)")
        if params.numel() != cursor:
            raise ValueError(f"shards cover {cursor} elements, the parameter vector has {params.numel()}")

        def cat(name: str, dim: int = 0):
            parts = [sd.get(name) for sd in by_begin]
            return None if any(p is None for p in parts) else torch.cat(parts, dim=dim)

        first = by_begin[0]
        return {"world": 1, "shard_begin": 0, "shard_len": cursor, "bounds": [0, cursor], "params": params, "m": cat("m"),
                "v": cat("v"), "master": cat("master"), "blt_state": cat("blt_state", 1), "toep_state": cat("toep_state", 1),
                "toep_pos": first.get("toep_pos", 0), "step_count": first["step_count"], "phi": first["phi"],
                "noise_key": first["noise_key"]}

    def _rotate(self, ptrs: list[int]) -> list[int]:
        """This rank's buffer first, then the peers starting at rank+1 (spreads NVLink traffic across peers)."""
        r = self.rank
        return [ptrs[(r + i) % len(ptrs)] for i in range(len(ptrs))]
