"""Native decoder runtime with an explicit backward that produces ONE example's gradient and its squared norm.

The reference obtains per-example gradients with ``vmap(grad)`` and materialises ``[microbatch, *P]``
(packages/opake-engine/src/opake/api/engine/clipping/_clipped_grad.py:278, _clipped_fun.py:805-850). For long
sequences (one example = one sequence of thousands of tokens) the B200 design instead runs each example through
ordinary tensor-core GEMMs with M = sequence length:

* the weight-gradient GEMM of every Linear writes the example's gradient tile (bf16) into a single reusable
  gradient buffer ``G`` and reduces ``sum(g^2)`` of the stored values in its epilogue, so the per-example norm costs
  no extra pass and no ``[B, *P]`` tensor ever exists;
* after the backward one tiny kernel turns the squared norm into the guarded clip factor and one bandwidth-bound
  kernel adds ``bf16(G * factor)`` to the fp32 clipped-gradient sum.

Shapes follow HuggingFace Llama / GPT-2 (fused QKV, interleaved gate/up rows); ``load_hf_state_dict`` converts names.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..ops import attention as A
from ..ops import gemm as G
from ..ops import kernels as K
from .config import DecoderConfig
from .flat import Layout, build_layout

_bf16 = torch.bfloat16


@dataclass
class ExampleStats:
    loss: torch.Tensor       # device scalar fp32
    n_tokens: torch.Tensor   # device scalar: number of supervised tokens


class DecoderRuntime:
    """Forward + per-example backward for dense decoders (Llama-style and GPT-2-style blocks)."""

    def __init__(self, cfg: DecoderConfig, params: torch.Tensor, *, layout: Layout | None = None,
                 attn_impl: str = "auto", n_slots: int = 1, wgrad_overlap: bool = True, ep=None,
                 canaries=None):
        if cfg.n_experts and (cfg.act != "swiglu" or cfg.n_experts > 256 or cfg.top_k > 32 or cfg.d_model % 8):
            raise ValueError("mixture-of-experts layers need SwiGLU experts, at most 256 experts and top_k <= 32")
        self.cfg = cfg
        # expert parallelism: an ``ExpertParallelRuntime`` that owns this rank's experts of every layer (the layout
        # then holds no expert matrices); ``None`` = all experts local, inside the flat parameter buffer
        self.ep = ep
        # a ``utils.CanaryPool``: gradient slots and workspaces are then allocated between guard bands (debugging aid)
        self.canaries = canaries
        self.layout = layout or build_layout(cfg, skip_experts=ep is not None)
        self.device = params.device
        self.params = params
        self.w = self.layout.views(params)
        # per-example gradient of the dense region (the token embedding is handled row-wise unless tied)
        # With two slots the clipped accumulation of example i can run on a side stream while example i+1 is
        # being computed into the other slot.
        self.n_slots = n_slots
        self.Gs = [self._alloc(self.layout.dense_total, dtype=_bf16, name=f"grad_slot{i}") for i in range(n_slots)]
        self.gs = [self.layout.views(G_, dense_only=True) for G_ in self.Gs]
        self.attn_impl = attn_impl
        self.sumsqs = [torch.zeros(1, dtype=torch.float64, device=self.device) for _ in range(n_slots)]
        self.scales = [torch.zeros(1, dtype=torch.float32, device=self.device) for _ in range(n_slots)]
        self.norms = [torch.zeros(1, dtype=torch.float32, device=self.device) for _ in range(n_slots)]
        self.clip_count = torch.zeros(1, dtype=torch.int32, device=self.device)
        self._ws: dict[int, dict] = {}
        self._rope = None
        # weights to pull from their owner during the NEXT forward pass (name -> the owner's copy, a peer-mapped
        # tensor): the consuming GEMM copies the matrix into this rank's replica band by band while it multiplies
        self._fetch: dict[str, torch.Tensor] | None = None
        self._stage_ready = torch.zeros(64, dtype=torch.int32, device=self.device) if self.device.type == "cuda" else None
        # Weight-gradient GEMMs run on a second stream next to the input-gradient GEMMs of the same layer: both are
        # persistent kernels that want every SM, so the second one's CTAs fill the SMs that the first one's last
        # (partial) wave of tiles leaves idle, and launch gaps disappear. ``wgrad_overlap=False`` keeps one stream.
        self._wstream = None
        if self.device.type == "cuda" and wgrad_overlap:
            self._wstream = torch.cuda.Stream(device=self.device)
        # small-vector gradients (norm weights, biases) are produced in fp32 rows and scattered into G at the end
        self._vec_names = [s.name for s in self.layout.slots
                           if len(s.shape) == 1 and s.offset < self.layout.dense_total]
        self._vec_row = {n: i for i, n in enumerate(self._vec_names)}
        d = cfg.d_model
        self._vec_width = max([d] + [self.layout.slot(n).numel for n in self._vec_names])
        self._n_leaves = len(self.layout.slots)
        self._widest = max(s.numel for s in self.layout.slots)

    # slot-0 aliases (single-buffer users and tests)
    @property
    def G(self):
        return self.Gs[0]

    @property
    def g(self):
        return self.gs[0]

    @property
    def sumsq(self):
        return self.sumsqs[0]

    @property
    def scale(self):
        return self.scales[0]

    @property
    def norm(self):
        return self.norms[0]

    def _alloc(self, *shape, dtype, name: str) -> torch.Tensor:
        if self.canaries is not None:
            return self.canaries.empty(*shape, dtype=dtype, name=name)
        return torch.empty(*shape, dtype=dtype, device=self.device)

    # ------------------------------------------------------------------ workspaces
    def workspace(self, T: int) -> dict:
        ws = self._ws.get(T)
        if ws is not None:
            return ws
        cfg, dev = self.cfg, self.device
        d, F, L = cfg.d_model, cfg.ffn, cfg.n_layers

        def e(*shape, dtype=_bf16):
            return self._alloc(*shape, dtype=dtype, name=f"workspace[T={T}]#{len(self.canaries) if self.canaries is not None else 0}")

        layers = []
        for _ in range(L):
            a = {"x": e(T, d), "xn": e(T, d), "qkv": e(T, cfg.qkv_dim), "attn": e(T, cfg.n_heads * cfg.head_dim),
                 "x_mid": e(T, d), "xn2": e(T, d)}
            if cfg.qk_norm:      # pre-normalisation queries and keys, needed by the norm's backward
                a["qk_raw"] = e(T, (cfg.n_heads + cfg.n_kv_heads) * cfg.head_dim)
                if cfg.qk_norm == "head":   # contiguous per-head rows: [T * heads, hd] views for the row kernels
                    a["q_raw"], a["k_raw"] = e(T, cfg.n_heads * cfg.head_dim), e(T, cfg.n_kv_heads * cfg.head_dim)
            if cfg.n_experts and self.ep is not None:
                pass        # token rows, pre-activations and routing state live in the expert-parallel layers
            elif cfg.n_experts:
                plan = K.MoePlan(T, cfg.n_experts, cfg.top_k, dev)
                I = cfg.expert_ffn
                a.update(plan=plan, rlogits=e(T, cfg.n_experts), xs=e(plan.R, d), gu=e(plan.R, 2 * I), act=e(plan.R, I),
                         ye=e(plan.R, d))
                # rows past the used segments are never written by the grouped GEMMs; keep them finite
                for name in ("gu", "act", "ye"):
                    a[name].zero_()
            elif cfg.act in ("swiglu", "geglu"):
                a["gu"], a["act"] = e(T, 2 * F), e(T, F)
            else:
                a["fc"], a["act"] = e(T, F), e(T, F)
            layers.append(a)
        tiles = G.lce_tiles(cfg.vocab_size)
        Vp = (cfg.vocab_size + 7) // 8 * 8
        ws = {
            "layers": layers, "x_last": e(T, d), "xf": e(T, d),
            "pmax": e(T, tiles, dtype=torch.float32), "psum": e(T, tiles, dtype=torch.float32),
            "tgt": e(T, dtype=torch.float32), "dlogits": e(T, Vp)[:, : cfg.vocab_size],
            "dx": e(T, d), "dx2": e(T, d), "dact": e(T, max(F, 8)), "dqkv": e(T, cfg.qkv_dim),
            "dwide": e(T, max(2 * F if cfg.act in ("swiglu", "geglu") else F, 8)),
            "dattn": e(T, cfg.n_heads * cfg.head_dim),
            "vec": torch.zeros(len(self._vec_names), self._vec_width, dtype=torch.float32, device=dev),
            "embs": [K.EmbeddingGradWorkspace(cfg.vocab_size, T, d, dev) for _ in range(self.n_slots)],
            "toks": [torch.zeros(T, dtype=torch.int32, device=dev) for _ in range(self.n_slots)],
            "labels": torch.zeros(T, dtype=torch.int32, device=dev),
            "loss": torch.zeros(1, dtype=torch.float32, device=dev), "ntok": torch.zeros(1, dtype=torch.float32, device=dev),
            "coef": torch.zeros(T, dtype=torch.float32, device=dev),
        }
        ws["vec_offsets"] = torch.tensor([self.layout.slot(n).offset for n in self._vec_names], dtype=torch.int64,
                                         device=dev)
        ws["emb"], ws["tok"] = ws["embs"][0], ws["toks"][0]
        if cfg.n_experts and self.ep is None:
            R, I = layers[0]["plan"].R, cfg.expert_ffn
            ws.update(dye=e(R, d), dgu=e(R, 2 * I).zero_(), dxs=e(R, d).zero_(),
                      dwts=e(T, cfg.top_k, dtype=torch.float32), drl=e(T, cfg.n_experts))
        self._ws[T] = ws
        return ws

    def _rope_table(self, T: int):
        cfg = self.cfg
        if self._rope is None or self._rope.shape[0] < T:
            self._rope = K.rope_table(max(T, cfg.max_seq), cfg.head_dim, cfg.rope_theta, device=self.device,
                                      scaling=cfg.rope_scaling)
        return self._rope

    def _vec(self, ws, name: str) -> torch.Tensor:
        n = self.layout.slot(name).numel
        return ws["vec"][self._vec_row[name], :n]

    # ------------------------------------------------------------------ second stream for weight gradients
    def _wgrad(self, dy, x, out, sumsq=None) -> None:
        """``out = dy^T x`` (+ squared norm) ordered after everything issued so far, on the weight-gradient stream."""
        side = self._wstream
        if side is None:
            G.linear_wgrad(dy, x, out=out, sumsq=sumsq)
            return
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            G.linear_wgrad(dy, x, out=out, sumsq=sumsq)

    def _wgrad_call(self, fn) -> None:
        """Runs ``fn`` (a weight-gradient launch) on the weight-gradient stream, ordered after everything issued so far."""
        side = self._wstream
        if side is None:
            fn()
            return
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            fn()

    def _wgrad_join(self) -> None:
        """Later work on the main stream (which may overwrite the operands) waits for the weight gradients issued so far."""
        if self._wstream is not None:
            torch.cuda.current_stream(self.device).wait_stream(self._wstream)

    # ------------------------------------------------------------------ norms
    def _norm_fwd(self, x, prefix: str, out=None):
        cfg, w = self.cfg, self.w
        if cfg.norm == "rms":
            y, rstd = K.rmsnorm_fwd(x, w[prefix + ".weight"], cfg.norm_eps, out=out)
            return y, (rstd,)
        y, mean, rstd = K.layernorm_fwd(x, w[prefix + ".weight"], w[prefix + ".bias"], cfg.norm_eps, out=out)
        return y, (mean, rstd)

    def _norm_bwd(self, ws, dy, x, prefix: str, stats, dres, out):
        cfg, w = self.cfg, self.w
        if cfg.norm == "rms":
            return K.rmsnorm_bwd(dy, x, w[prefix + ".weight"], stats[0], dres=dres, dw=self._vec(ws, prefix + ".weight"),
                                 out=out)
        return K.layernorm_bwd(dy, x, w[prefix + ".weight"], stats[0], stats[1], dres=dres,
                               dw=self._vec(ws, prefix + ".weight"), db=self._vec(ws, prefix + ".bias"), out=out)

    def _wop(self, name: str):
        """Operand and staging arguments of a forward GEMM on weight ``name``: the local replica, or (when the engine
        marked the weight for fetching) the owner's copy together with the replica as the staging destination."""
        src = self._fetch.get(name) if self._fetch else None
        if src is None:
            return self.w[name], None
        return src, (self.w[name], self._stage_ready)

    @staticmethod
    def stageable(name: str, shape: tuple, T: int, act: str) -> bool:
        """Whether the forward GEMM that consumes weight ``name`` can fetch it from another GPU while it multiplies:
        plain or SwiGLU epilogue, at least 256 rows and more than 128 columns (the two-CTA kernel), 16-byte rows."""
        leaf = name.rsplit(".", 1)[-1]
        if leaf not in ("wqkv", "wo", "wgu", "wd", "wfc", "wproj") or len(shape) != 2:
            return False
        n, k = shape
        return T >= 256 and n > 128 and n % 8 == 0 and k % 8 == 0 and G.pair_mode()

    # ------------------------------------------------------------------ forward
    def forward(self, tok: torch.Tensor, labels: torch.Tensor | None, ws: dict | None = None):
        """Runs the decoder on one sequence. Returns ``(per-token nll [T], lse, saved)``.

        ``labels`` are already shifted (``labels[t]`` is the target of position ``t``; negative = ignored).
        """
        cfg, w = self.cfg, self.w
        T = tok.numel()
        ws = ws or self.workspace(T)
        H, KV, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        x = K.embedding_fwd(tok, w["embed"], w.get("wpe") if cfg.pos == "learned" else None, out=ws["layers"][0]["x"])
        saved = []
        for li in range(cfg.n_layers):
            a = ws["layers"][li]
            p = f"layers.{li}."
            xn, st1 = self._norm_fwd(x, p + "norm1", out=a["xn"])
            wsrc, stg = self._wop(p + "wqkv")
            G.gemm(xn, wsrc, out=a["qkv"], bias=w.get(p + "bqkv"), stage=stg)
            stq = None
            if cfg.qk_norm == "head":
                nq, nk = H * hd, KV * hd
                a["q_raw"].copy_(a["qkv"][:, :nq])
                a["k_raw"].copy_(a["qkv"][:, nq : nq + nk])
                qn, rq = K.rmsnorm_fwd(a["q_raw"].view(T * H, hd), w[p + "q_norm.weight"], cfg.norm_eps,
                                       out=a["qk_raw"].view(-1)[: T * nq].view(T * H, hd))
                kn, rk = K.rmsnorm_fwd(a["k_raw"].view(T * KV, hd), w[p + "k_norm.weight"], cfg.norm_eps,
                                       out=a["qk_raw"].view(-1)[T * nq : T * (nq + nk)].view(T * KV, hd))
                a["qkv"][:, :nq].copy_(qn.view(T, nq))
                a["qkv"][:, nq : nq + nk].copy_(kn.view(T, nk))
                stq = (rq, rk)
            elif cfg.qk_norm:
                nq, nk = H * hd, KV * hd
                a["qk_raw"].copy_(a["qkv"][:, : nq + nk])
                _, rq = K.rmsnorm_fwd(a["qk_raw"][:, :nq], w[p + "q_norm.weight"], cfg.norm_eps, out=a["qkv"][:, :nq])
                _, rk = K.rmsnorm_fwd(a["qk_raw"][:, nq:], w[p + "k_norm.weight"], cfg.norm_eps, out=a["qkv"][:, nq : nq + nk])
                stq = (rq, rk)
            if cfg.pos == "rope":
                K.rope_(a["qkv"], self._rope_table(T), H + KV, hd)
            _, actx = A.attention_fwd(a["qkv"], H, KV, hd, self.attn_impl, out=a["attn"])
            # output projection with the residual add fused into the GEMM epilogue
            wsrc, stg = self._wop(p + "wo")
            G.gemm(a["attn"], wsrc, out=a["x_mid"], residual=x, bias=w.get(p + "bo"), stage=stg)
            xn2, st2 = self._norm_fwd(a["x_mid"], p + "norm2", out=a["xn2"])
            nxt = ws["layers"][li + 1]["x"] if li + 1 < cfg.n_layers else ws["x_last"]
            if cfg.n_experts and self.ep is not None:
                self.ep.forward(li, xn2, a["x_mid"], nxt)
            elif cfg.n_experts:
                plan = a["plan"]
                G.gemm(xn2, w[p + "router"], out=a["rlogits"])
                K.moe_route(a["rlogits"], plan, cfg.norm_topk_prob)
                K.moe_gather(xn2, plan, a["xs"])
                G.gemm(a["xs"], w[p + "experts.wgu"], out=a["gu"], epilogue=G.EPI_SWIGLU, act=a["act"], tile_group=plan.tile_group)
                G.gemm(a["act"], w[p + "experts.wd"], out=a["ye"], tile_group=plan.tile_group)
                K.moe_combine(a["ye"], plan, nxt, wts=plan.wts, residual=a["x_mid"])
            elif cfg.act == "swiglu":
                wsrc, stg = self._wop(p + "wgu")
                G.gemm(xn2, wsrc, out=a["gu"], epilogue=G.EPI_SWIGLU, act=a["act"], stage=stg)
                wsrc, stg = self._wop(p + "wd")
                G.gemm(a["act"], wsrc, out=nxt, residual=a["x_mid"], stage=stg)
            elif cfg.act == "geglu":
                wsrc, stg = self._wop(p + "wgu")
                G.gemm(xn2, wsrc, out=a["gu"], stage=stg)
                K.geglu_fwd(a["gu"], True, out=a["act"])
                wsrc, stg = self._wop(p + "wd")
                G.gemm(a["act"], wsrc, out=nxt, residual=a["x_mid"], stage=stg)
            else:
                wsrc, stg = self._wop(p + "wfc")
                G.gemm(xn2, wsrc, out=a["fc"], bias=w.get(p + "bfc"), stage=stg)
                K.gelu_fwd(a["fc"], out=a["act"])
                wsrc, stg = self._wop(p + "wproj")
                G.gemm(a["act"], wsrc, out=nxt, residual=a["x_mid"], bias=w.get(p + "bproj"), stage=stg)
            saved.append((st1, st2, actx, stq))
            x = nxt
        xf, stf = self._norm_fwd(x, "norm_f", out=ws["xf"])
        head = w["embed"] if cfg.tie_embeddings else w["lm_head"]
        nll = lse = None
        if labels is not None:
            G.gemm(xf, head, epilogue=G.EPI_LCE_FWD, labels=labels, pmax=ws["pmax"], psum=ws["psum"], tgt=ws["tgt"])
            lse, nll = K.lce_finalize(ws["pmax"], ws["psum"], ws["tgt"], labels)
        return nll, lse, (saved, stf)

    def logits(self, tok: torch.Tensor) -> torch.Tensor:
        """Full ``[T, V]`` logits (evaluation / generation path)."""
        ws = self.workspace(tok.numel())
        self.forward(tok, None, ws)
        head = self.w["embed"] if self.cfg.tie_embeddings else self.w["lm_head"]
        Vp = (self.cfg.vocab_size + 7) // 8 * 8
        out = torch.empty(tok.numel(), Vp, dtype=_bf16, device=self.device)[:, : self.cfg.vocab_size]
        return G.gemm(ws["xf"], head, out=out)

    # ------------------------------------------------------------------ forward + backward of one example
    def example_grad(self, tok: torch.Tensor, labels: torch.Tensor, *, loss_weight: torch.Tensor | None = None,
                     ws: dict | None = None, slot: int = 0, before_wgrad=None) -> ExampleStats:
        """Computes this example's gradient into ``self.G`` (+ compact embedding rows) and ``sumsq``.

        ``before_wgrad`` (optional callable) runs once, after the forward pass and right before the first kernel that
        writes the slot's gradient buffer: the place to wait for a consumer of the buffer's previous contents.

        The example loss is the mean NLL over supervised tokens (per-example divisor, as
        packages/opake-alignment/src/opake/api/alignment/sft/loss/_nll.py:43-88).
        """
        cfg, w, g = self.cfg, self.w, self.gs[slot]
        sumsq, emb_ws = self.sumsqs[slot], None
        T = tok.numel()
        ws = ws or self.workspace(T)
        emb_ws = ws["embs"][slot]
        H, KV, hd = cfg.n_heads, cfg.n_kv_heads, cfg.head_dim
        nll, lse, (saved, stf) = self.forward(tok, labels, ws)
        coef, loss, ntok = ws["coef"], ws["loss"], ws["ntok"]
        K.loss_coef(labels, nll, coef, loss, ntok, weight=loss_weight)
        ws["vec"].zero_()
        sumsq.zero_()

        head = w["embed"] if cfg.tie_embeddings else w["lm_head"]
        ghead = g["embed"] if cfg.tie_embeddings else g["lm_head"]
        dlog = G.gemm(ws["xf"], head, out=ws["dlogits"], epilogue=G.EPI_LCE_BWD, labels=labels, lse=lse, coef=coef)
        if before_wgrad is not None:
            before_wgrad()
        if cfg.tie_embeddings:
            self._wgrad(dlog, ws["xf"], ghead)                   # norm added after the embedding rows are merged
        else:
            self._wgrad(dlog, ws["xf"], ghead, sumsq)
        dxf = G.gemm(dlog, head, b_mn=True, out=ws["dx2"])
        x_last = ws["x_last"]
        dx = self._norm_bwd(ws, dxf, x_last, "norm_f", stf, None, ws["dx"])

        for li in reversed(range(cfg.n_layers)):
            a = ws["layers"][li]
            p = f"layers.{li}."
            st1, st2, actx, stq = saved[li]
            # ---- MLP
            if cfg.n_experts and self.ep is not None:
                # expert parallel: rows travel to the experts' owners; only squared norms of the expert gradients are
                # formed in this pass, the router gradient is this rank's own
                dxn2 = self.ep.backward(li, dx, router_grad_out=g[p + "router"], sumsq=sumsq, dx_out=ws["dx2"])
            elif cfg.n_experts:
                plan = a["plan"]
                K.moe_combine_bwd(dx, a["ye"], plan, ws["dwts"])
                K.moe_gather(dx, plan, ws["dye"], entry_scale=plan.wts)
                # expert weight gradients: one grouped GEMM per matrix, reduction range of expert e = its row segment
                self._wgrad_call(lambda: G.gemm(ws["dye"], a["act"], a_mn=True, b_mn=True, out=g[p + "experts.wd"],
                                                epilogue=G.EPI_SUMSQ, sumsq=sumsq, group_k=plan.group_k, sumsq_shared=True))
                G.swiglu_dgrad(ws["dye"], w[p + "experts.wd"], a["gu"], out=ws["dgu"], tile_group=plan.tile_group)
                self._wgrad_call(lambda: G.gemm(ws["dgu"], a["xs"], a_mn=True, b_mn=True, out=g[p + "experts.wgu"],
                                                epilogue=G.EPI_SUMSQ, sumsq=sumsq, group_k=plan.group_k, sumsq_shared=True))
                G.gemm(ws["dgu"], w[p + "experts.wgu"], b_mn=True, out=ws["dxs"], tile_group=plan.tile_group)
                dxn2 = K.moe_combine(ws["dxs"], plan, ws["dx2"])
                # router: d weights -> d logits -> router weight gradient and the second path into dxn2
                K.moe_route_bwd(plan, ws["dwts"], ws["drl"], cfg.norm_topk_prob)
                G.linear_wgrad(ws["drl"], a["xn2"], out=g[p + "router"], sumsq=sumsq)
                G.gemm(ws["drl"], w[p + "router"], b_mn=True, out=dxn2, residual=dxn2)
                self._wgrad_join()            # dye / dgu are rewritten by the next layer, dx by the norm backward below
            elif cfg.act in ("swiglu", "geglu"):
                self._wgrad(dx, a["act"], g[p + "wd"], sumsq)
                dgu = ws["dwide"]
                if cfg.act == "swiglu":       # d(act) stays in the accumulator: SwiGLU backward runs in the dgrad epilogue
                    G.swiglu_dgrad(dx, w[p + "wd"], a["gu"], out=dgu)
                else:
                    dact = G.gemm(dx, w[p + "wd"], b_mn=True, out=ws["dact"])
                    K.geglu_bwd(dact, a["gu"], True, out=dgu)
                self._wgrad(dgu, a["xn2"], g[p + "wgu"], sumsq)
                dxn2 = G.gemm(dgu, w[p + "wgu"], b_mn=True, out=ws["dx2"])
                self._wgrad_join()            # the norm backward below overwrites dx in place
            else:
                G.linear_wgrad(dx, a["act"], out=g[p + "wproj"], sumsq=sumsq)
                if cfg.bias:
                    K.colsum_(dx, self._vec(ws, p + "bproj"))
                dact = G.gemm(dx, w[p + "wproj"], b_mn=True, out=ws["dact"])
                dfc = K.gelu_bwd(dact, a["fc"], out=ws["dwide"])
                G.linear_wgrad(dfc, a["xn2"], out=g[p + "wfc"], sumsq=sumsq)
                if cfg.bias:
                    K.colsum_(dfc, self._vec(ws, p + "bfc"))
                dxn2 = G.gemm(dfc, w[p + "wfc"], b_mn=True, out=ws["dx2"])
            dx_mid = self._norm_bwd(ws, dxn2, a["x_mid"], p + "norm2", st2, dx, ws["dx"])  # in place over dres
            # ---- attention
            self._wgrad(dx_mid, a["attn"], g[p + "wo"], sumsq)
            if cfg.bias:
                K.colsum_(dx_mid, self._vec(ws, p + "bo"))
            dattn = G.gemm(dx_mid, w[p + "wo"], b_mn=True, out=ws["dattn"])
            dqkv = ws["dqkv"]
            A.attention_bwd(dattn, a["qkv"], a["attn"], actx, H, KV, hd, dqkv)
            if cfg.pos == "rope":
                K.rope_(dqkv, self._rope_table(T), H + KV, hd, backward=True)
            if cfg.qk_norm == "head":
                nq, nk = H * hd, KV * hd
                dq_c = a["qk_raw"].view(-1)[: T * nq].view(T, nq)           # the normalised copies are dead by now
                dk_c = a["qk_raw"].view(-1)[T * nq : T * (nq + nk)].view(T, nk)
                dq_c.copy_(dqkv[:, :nq])
                dk_c.copy_(dqkv[:, nq : nq + nk])
                K.rmsnorm_bwd(dq_c.view(T * H, hd), a["q_raw"].view(T * H, hd), w[p + "q_norm.weight"], stq[0],
                              dw=self._vec(ws, p + "q_norm.weight"), out=dq_c.view(T * H, hd))
                K.rmsnorm_bwd(dk_c.view(T * KV, hd), a["k_raw"].view(T * KV, hd), w[p + "k_norm.weight"], stq[1],
                              dw=self._vec(ws, p + "k_norm.weight"), out=dk_c.view(T * KV, hd))
                dqkv[:, :nq].copy_(dq_c)
                dqkv[:, nq : nq + nk].copy_(dk_c)
            elif cfg.qk_norm:      # in place on the query and key columns of dqkv
                nq, nk = H * hd, KV * hd
                K.rmsnorm_bwd(dqkv[:, :nq], a["qk_raw"][:, :nq], w[p + "q_norm.weight"], stq[0],
                              dw=self._vec(ws, p + "q_norm.weight"), out=dqkv[:, :nq])
                K.rmsnorm_bwd(dqkv[:, nq : nq + nk], a["qk_raw"][:, nq:], w[p + "k_norm.weight"], stq[1],
                              dw=self._vec(ws, p + "k_norm.weight"), out=dqkv[:, nq : nq + nk])
            self._wgrad(dqkv, a["xn"], g[p + "wqkv"], sumsq)
            if cfg.bias or cfg.qkv_bias:
                K.colsum_(dqkv, self._vec(ws, p + "bqkv"))
            dxn = G.gemm(dqkv, w[p + "wqkv"], b_mn=True, out=ws["dx2"])
            self._wgrad_join()                # dx_mid (read by the wo gradient) is overwritten in place below
            dx = self._norm_bwd(ws, dxn, a["x"], p + "norm1", st1, dx_mid, ws["dx"])

        self._wgrad_join()
        # ---- embeddings
        K.embedding_bwd_compact(tok, dx, emb_ws, None if cfg.tie_embeddings else sumsq)
        if cfg.pos == "learned":
            gw = g["wpe"]
            gw[:T].copy_(dx)
            gw[T:].zero_()
            K.sumsq_(gw[:T], sumsq)
        if cfg.tie_embeddings:
            K.embedding_add_rows(tok, emb_ws, ghead, T)
            K.sumsq_(ghead, sumsq)
        # ---- vector parameters (norm weights, biases): fp32 rows -> bf16 slots of G, with their norm
        if all(self.layout.slot(n).numel == self._vec_width for n in self._vec_names):
            K.scatter_rows_cast_sumsq(ws["vec"], self.Gs[slot], ws["vec_offsets"], sumsq)
        else:
            self._scatter_vec_rows(ws, slot)
        return ExampleStats(loss=loss, n_tokens=ntok)

    def _scatter_vec_rows(self, ws, slot: int = 0) -> None:
        for n in self._vec_names:
            row = self._vec(ws, n)
            dst = self.gs[slot][n]
            K.cast_f32_bf16(row, dst)
            K.sumsq_(dst, self.sumsqs[slot])

    # ------------------------------------------------------------------ clip + accumulate
    def clip_factor(self, clip: float, *, auto: bool = False, gamma: float = 0.01, slot: int = 0) -> None:
        """Turns the slot's squared norm into the guarded clip factor (device scalar) and resets the accumulator."""
        K.clip_scale(self.sumsqs[slot], clip, scale_out=self.scales[slot], norm_out=self.norms[slot],
                     counters=self.clip_count, auto=auto, gamma=gamma, n_leaves=self._n_leaves,
                     widest_leaf=self._widest, reset=True)

    def accumulate(self, acc: torch.Tensor, ws: dict, tok: torch.Tensor, *, slot: int = 0, overwrite: bool = False) -> None:
        """``acc`` (fp32, full flat layout) ``+= clip_factor * G[slot]`` with the conservative storage rounding."""
        K.clip_accumulate(self.Gs[slot], self.scales[slot], acc[: self.layout.dense_total], overwrite=overwrite)
        if not self.cfg.tie_embeddings:
            emb = self.layout.slot("embed")
            acc_emb = acc[emb.offset : emb.offset + emb.numel].view(emb.shape)
            K.embedding_accumulate(tok, ws["embs"][slot], self.scales[slot], acc_emb, tok.numel())

    def accumulate_group(self, acc: torch.Tensor, ws: dict, n: int, *, overwrite: bool = False, toks=None) -> None:
        """Adds the clipped gradients of the examples held in slots ``0 .. n-1`` in one pass over ``acc``: the fp32
        sums are read and written once for the whole group. ``toks``: the token tensors of the slots when they are not
        ``ws["toks"]`` any more (a slot's token buffer is refilled before a deferred accumulation runs)."""
        K.clip_accumulate_group(self.Gs[:n], self.scales[:n], acc[: self.layout.dense_total], overwrite=overwrite)
        if not self.cfg.tie_embeddings:
            emb = self.layout.slot("embed")
            acc_emb = acc[emb.offset : emb.offset + emb.numel].view(emb.shape)
            for j in range(n):
                tok = ws["toks"][j] if toks is None else toks[j]
                K.embedding_accumulate(tok, ws["embs"][j], self.scales[j], acc_emb, tok.numel())

    def accumulate_group_sharded(self, acc_ptrs: list[int], bounds: list[int], rank: int, ws: dict, n: int, *,
                                 emb_acc: torch.Tensor | None, toks=None) -> None:
        """Sharded sums: the clipped gradients of the examples in slots ``0 .. n-1`` are reduced into the owners' fp32
        shards (``acc_ptrs`` / ``bounds`` as in ``ops.kernels.clip_accumulate_group_push``). ``emb_acc``: the ``[V, d]``
        rows of the embedding table's sum inside its owner's shard (possibly on another GPU)."""
        K.clip_accumulate_group_push(self.Gs[:n], self.scales[:n], acc_ptrs, bounds, rank, self.layout.dense_total)
        if not self.cfg.tie_embeddings and emb_acc is not None:
            for j in range(n):
                tok = ws["toks"][j] if toks is None else toks[j]
                K.embedding_accumulate(tok, ws["embs"][j], self.scales[j], emb_acc, tok.numel(), shared=True)

    def clip_and_accumulate(self, acc: torch.Tensor, clip: float, ws: dict, tok: torch.Tensor, *, auto: bool = False,
                            gamma: float = 0.01, overwrite: bool = False, slot: int = 0) -> None:
        self.clip_factor(clip, auto=auto, gamma=gamma, slot=slot)
        self.accumulate(acc, ws, tok, slot=slot, overwrite=overwrite)


def expert_seed(seed: int, layer: int, expert: int) -> int:
    """Seed of one expert's initial weights: a function of the GLOBAL expert id, so the model is the same whether its
    experts sit in one flat buffer or are spread over expert-parallel ranks."""
    return seed * 1_000_003 + layer * 4099 + expert + 1


def init_expert_(wgu: torch.Tensor, wd: torch.Tensor, seed: int, layer: int, expert: int, n_layers: int, std: float = 0.02) -> None:
    gen = torch.Generator(device=wgu.device).manual_seed(expert_seed(seed, layer, expert))
    wgu.copy_(torch.randn(wgu.shape, generator=gen, device=wgu.device, dtype=torch.float32) * std)
    wd.copy_(torch.randn(wd.shape, generator=gen, device=wd.device, dtype=torch.float32) * (std / (2 * n_layers) ** 0.5))


def init_params_(cfg: DecoderConfig, params: torch.Tensor, layout: Layout, seed: int = 0, std: float = 0.02) -> None:
    """Random-normal weights (std 0.02, output projections scaled by 1/sqrt(2L)), unit norm weights, zero biases.
    Every tensor draws from its own generator, seeded by the tensor's name: the values do not depend on which other
    tensors the layout holds (expert matrices may live elsewhere under expert parallelism)."""
    import zlib

    params.zero_()
    for s in layout.slots:
        v = params[s.offset : s.offset + s.numel]
        if s.name.endswith(("norm1.weight", "norm2.weight", "q_norm.weight", "k_norm.weight")) or s.name == "norm_f.weight":
            v.fill_(1.0)
        elif len(s.shape) == 1:
            v.zero_()
        elif s.name.endswith("experts.wgu"):
            li = int(s.name.split(".")[1])
            wd_slot = layout.slot(s.name[: -len("wgu")] + "wd")
            wd_all = params[wd_slot.offset : wd_slot.offset + wd_slot.numel].view(wd_slot.shape)
            wgu_all = v.view(s.shape)
            for e in range(s.shape[0]):
                init_expert_(wgu_all[e], wd_all[e], seed, li, e, cfg.n_layers, std)
        elif s.name.endswith("experts.wd"):
            continue            # filled together with the gate / up matrices above
        else:
            scale = std
            if s.name.endswith(("wo", "wd", "wproj")):
                scale = std / (2 * cfg.n_layers) ** 0.5
            gen = torch.Generator(device=params.device).manual_seed((seed * 2654435761 + zlib.crc32(s.name.encode())) & 0x7FFFFFFFFFFFFFFF)
            # chunked fill keeps the fp32 temporary small for multi-GB tensors
            step = 1 << 26
            for b in range(0, s.numel, step):
                n = min(step, s.numel - b)
                v[b : b + n].copy_(torch.randn(n, generator=gen, device=params.device, dtype=torch.float32) * scale)
