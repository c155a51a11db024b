"""Device-resident weights of a decoder stack in the layouts the kernels read.

Layouts (all ``[out, in]`` = checkpoint order, bf16):

* ``wqkv``  fused ``[q heads | k heads | v heads]`` rows (the reference keeps Q, K, V separate,
  crates/poot-models/tests/launch_census/real_dims.tsv:69-72; fusing saves two launches per layer).
* ``wgu``   gate and up rows interleaved (row ``2j`` = gate_j, row ``2j+1`` = up_j) so SwiGLU runs in the GEMM /
  GEMV epilogue on adjacent accumulators.
* tensor-parallel rank views follow the Megatron layouts of the reference's ``shard``
  (crates/poot-graph-plan/src/passes/sharding.rs:219-251): q/k/v/gate/up split on ``out``, o/down split on ``in``,
  embedding, head and norms replicated.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Dict, List, Optional

import torch

from ..models.config import DecoderConfig


@dataclass
class LayerWeights:
    ln1: torch.Tensor
    ln2: torch.Tensor
    wqkv: torch.Tensor
    wo: torch.Tensor
    wgu: Optional[torch.Tensor] = None      # dense FFN
    wdown: Optional[torch.Tensor] = None
    q_norm: Optional[torch.Tensor] = None
    k_norm: Optional[torch.Tensor] = None
    bqkv: Optional[torch.Tensor] = None     # fused q|k|v bias of families that have one (qwen2), rank-local
    post1: Optional[torch.Tensor] = None    # norm applied to the attention output before the residual add (post / sandwich blocks)
    post2: Optional[torch.Tensor] = None    # the same for the FFN output
    wgate: Optional[torch.Tensor] = None    # attention output gate projection [q_size, hidden] (gated attention)
    bo: Optional[torch.Tensor] = None       # bias of the attention output projection
    ln1_b: Optional[torch.Tensor] = None    # LayerNorm biases (families whose norms carry one)
    ln2_b: Optional[torch.Tensor] = None
    bgu: Optional[torch.Tensor] = None      # dense FFN biases: gate/up (interleaved like wgu, or up only) and down
    bdown: Optional[torch.Tensor] = None
    sinks: Optional[torch.Tensor] = None    # [heads] fp32 sink logits joining every softmax denominator
    router_bias: Optional[torch.Tensor] = None    # [E] fp32 added to the router logits
    ex_bgu: Optional[torch.Tensor] = None   # [E, 2F] expert gate/up biases in the interleaved row order of ex_wgu
    ex_bdown: Optional[torch.Tensor] = None  # [E, hidden] expert down-projection biases
    kind: str = "attention"                 # token mixer of the layer: attention | gdn | mla | mamba | none (FFN-only block)
    ssm: Optional[Dict[str, torch.Tensor]] = None   # Mamba2: conv [C, K], conv_bias, dt_bias, a_log, d (fp32), gate_norm (bf16)
    mla: Optional[Dict[str, torch.Tensor]] = None   # latent attention: q_a, q_a_norm, q_b (or q), kv_a, kv_a_norm, kv_b
    gdn: Optional[Dict[str, torch.Tensor]] = None   # gated delta net: w_in (q|k|v|z|b|a rows), conv [C, K], dt_bias, a_log, gate_norm
    router: Optional[torch.Tensor] = None   # [E, hidden]
    select_bias: Optional[torch.Tensor] = None   # [E] fp32, added to the router scores for selection only
    sh_wgu: Optional[torch.Tensor] = None   # always-on (shared) expert: interleaved gate/up rows, down projection
    sh_wdown: Optional[torch.Tensor] = None
    sh_gate: Optional[torch.Tensor] = None  # [8, hidden]: row 0 is the shared expert's sigmoid gate, the rest zero padding
    ex_packed: Optional[object] = None      # ``ops.cuda_ops.PackedExperts``: the routed experts as stored (then ex_wgu / ex_wdown are unset)
    ex_wgu: Optional[torch.Tensor] = None   # [E_local, 2F, hidden]
    ex_wdown: Optional[torch.Tensor] = None  # [E_local, hidden, F]
    quant: Dict[str, object] = field(default_factory=dict)  # packed (GGUF block) weights by role


@dataclass(frozen=True)
class StageSpec:
    """One stage of a layer pipeline: layers ``[l0, l1)`` of the model on this rank; the token embedding lives on the
    first stage, the final norm and the head on the last (crates/poot-llm/src/driver/placement.rs:1-16)."""
    index: int
    count: int
    l0: int
    l1: int

    @property
    def first(self) -> bool:
        return self.index == 0

    @property
    def last(self) -> bool:
        return self.index == self.count - 1

    @staticmethod
    def whole(cfg: DecoderConfig) -> "StageSpec":
        return StageSpec(0, 1, 0, cfg.n_layers)


@dataclass
class DecoderWeights:
    cfg: DecoderConfig
    embed: torch.Tensor
    final_norm: torch.Tensor
    lm_head: torch.Tensor
    layers: List[LayerWeights]
    tp_rank: int = 0
    tp_world: int = 1
    ep_rank: int = 0        # expert-parallel share: this rank holds experts [ep_rank * E/ep_world, ...)
    ep_world: int = 1
    quant: Dict[str, object] = field(default_factory=dict)
    stage: Optional[StageSpec] = None      # None = the whole model; else ``layers`` holds layers [stage.l0, stage.l1)
    final_norm_b: Optional[torch.Tensor] = None
    embed_norm: Optional[torch.Tensor] = None     # LayerNorm right after the embedding (bloom), with its bias
    embed_norm_b: Optional[torch.Tensor] = None
    # a multi-token-prediction layer's input side: {"enorm", "hnorm"} norm weights and the two halves of its projection
    # {"we": eh_proj[:, :H] over the token embedding, "wh": eh_proj[:, H:] over the hidden-state carry}
    mtp: Optional[Dict[str, torch.Tensor]] = None

    @property
    def layer0(self) -> int:
        return 0 if self.stage is None else self.stage.l0

    def nbytes(self) -> int:
        n = 0
        seen = set()

        def add(t):
            nonlocal n
            if hasattr(t, "packed"):          # block-quantised weight
                t = t.packed
            if isinstance(t, torch.Tensor) and t.data_ptr() not in seen:
                seen.add(t.data_ptr())
                n += t.numel() * t.element_size()

        for t in (self.embed, self.final_norm, self.lm_head):
            if t is not None:
                add(t)
        for L in self.layers:
            for v in vars(L).values():
                add(v)
        return n


class UnsupportedOnDevice(ValueError):
    """The configuration uses a feature the device program does not implement."""


def fold_scales(w: "DecoderWeights") -> "DecoderWeights":
    """Fold the constant multipliers of a family into the weights they multiply, so the device program needs no extra
    work per token: ``residual_scale`` (Granite) into the o / down projections, ``logit_scale`` into the LM head
    (on a private copy when the head is tied to the embedding).  ``embed_scale`` stays a runtime multiply because a
    tied head must see the unscaled table."""
    cfg = w.cfg
    if getattr(w, "_scales_folded", False):
        return w
    if cfg.residual_scale != 1.0 and cfg.block != "pre":
        raise UnsupportedOnDevice("residual_scale with a norm between the projection and the residual add")
    if cfg.residual_scale != 1.0:
        for L in w.layers:
            for role in ("wo", "wdown", "ex_wdown"):
                t = getattr(L, role)
                if t is None:
                    continue
                if not isinstance(t, torch.Tensor):
                    raise UnsupportedOnDevice("residual_scale cannot be folded into block-quantised projections")
                setattr(L, role, (t.float() * cfg.residual_scale).to(t.dtype))
    if cfg.logit_scale != 1.0 and w.lm_head is not None:
        if not isinstance(w.lm_head, torch.Tensor):
            raise UnsupportedOnDevice("logit_scale cannot be folded into a block-quantised LM head")
        w.lm_head = (w.lm_head.float() * cfg.logit_scale).to(w.lm_head.dtype)     # a new tensor: a tied table stays as is
    w._scales_folded = True
    return w


def fuse_qkv_bias(bq: torch.Tensor, bk: torch.Tensor, bv: torch.Tensor, cfg: DecoderConfig, rank: int = 0,
                  world: int = 1) -> torch.Tensor:
    """Rank-local fused bias in the row order of :func:`fuse_qkv`."""
    return fuse_qkv(bq[:, None], bk[:, None], bv[:, None], cfg, rank, world)[:, 0].contiguous()


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``[F, H]`` gate and up -> ``[2F, H]`` with rows (gate_0, up_0, gate_1, up_1, ...)."""
    F, H = gate.shape
    return torch.stack([gate, up], dim=1).reshape(2 * F, H).contiguous()


def shard_rows(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[0] // world
    return w[rank * n:(rank + 1) * n].contiguous()


def shard_cols(w: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    n = w.shape[1] // world
    return w[:, rank * n:(rank + 1) * n].contiguous()


def fuse_qkv(wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor, cfg: DecoderConfig, rank: int = 0,
             world: int = 1) -> torch.Tensor:
    """Fused, rank-local QKV: this rank's query heads, then its KV heads."""
    D = cfg.head_dim
    hq, hkv = cfg.n_heads // world, max(cfg.n_kv_heads // world, 1)
    q = wq[rank * hq * D:(rank + 1) * hq * D]
    # first KV head of this rank; with fewer KV heads than ranks a head is replicated over world/n_kv ranks
    k0 = rank * hkv if cfg.n_kv_heads >= world else rank * cfg.n_kv_heads // world
    k = wk[k0 * D:(k0 + hkv) * D]
    v = wv[k0 * D:(k0 + hkv) * D]
    return torch.cat([q, k, v], dim=0).contiguous()


def mtp_input_weights(enorm: torch.Tensor, hnorm: torch.Tensor, eh_proj: torch.Tensor) -> Dict[str, torch.Tensor]:
    """The input side of a multi-token-prediction layer in the engine's layout: ``eh_proj[H, 2H]`` multiplies
    ``[enorm(embedding) ; hnorm(carry)]``; it is kept as its two halves so the concatenation never materialises."""
    H = eh_proj.shape[0]
    return {"enorm": enorm.contiguous(), "hnorm": hnorm.contiguous(), "we": eh_proj[:, :H].contiguous(),
            "wh": eh_proj[:, H:].contiguous()}


def share_tables(layer: DecoderWeights, target: DecoderWeights) -> DecoderWeights:
    """A multi-token-prediction layer embeds and un-embeds with the target's own tables (no second copy on the device)."""
    layer.embed, layer.lm_head = target.embed, target.lm_head
    return layer


def random_weights(cfg: DecoderConfig, device, seed: int = 0, std: float = 0.02, tp_rank: int = 0, tp_world: int = 1,
                   ep_rank: int = 0, ep_world: int = 1, dtype=torch.bfloat16, stage: Optional[StageSpec] = None) -> DecoderWeights:
    """Random-init weights ``~N(0, std)`` generated directly in the rank-local fused layouts.

    Each tensor is drawn from a generator seeded by (seed, layer, role) so a rank's shard of a weight equals the
    same slice of the weight any other world size would draw: TP=1 and TP=8 runs compute the same model.
    """
    dev = torch.device(device)
    H, D = cfg.hidden, cfg.head_dim

    def draw(shape, tag: int):
        g = torch.Generator(device=dev)
        g.manual_seed((seed * 1000003 + tag) & 0x7fffffff)
        return (torch.randn(shape, generator=g, device=dev, dtype=torch.float32) * std).to(dtype)

    def ones(n):
        return torch.ones(n, dtype=dtype, device=dev)

    layers = []
    st = stage or StageSpec.whole(cfg)
    for l in range(st.l0, st.l1):
        t = (l + 1) * 64
        wq = draw((cfg.q_size, H), t + 0)
        wk = draw((cfg.kv_size, H), t + 1)
        wv = draw((cfg.kv_size, H), t + 2)
        wqkv = fuse_qkv(wq, wk, wv, cfg, tp_rank, tp_world)
        del wq, wk, wv
        wo = shard_cols(draw((H, cfg.q_size), t + 3), tp_rank, tp_world)
        L = LayerWeights(ln1=ones(H), ln2=ones(H), wqkv=wqkv, wo=wo)
        if cfg.attn_bias:
            L.bqkv = fuse_qkv_bias(draw((cfg.q_size,), t + 60), draw((cfg.kv_size,), t + 61), draw((cfg.kv_size,), t + 62),
                                   cfg, tp_rank, tp_world)
        if cfg.qk_norm:
            L.q_norm, L.k_norm = ones(D), ones(D)
        if cfg.is_moe:
            F = cfg.moe_ffn
            L.router = draw((cfg.n_experts, H), t + 4)
            e_local = cfg.n_experts // ep_world
            gus, downs = [], []
            for e in range(ep_rank * e_local, (ep_rank + 1) * e_local):
                g_ = draw((F, H), t + 8 + 3 * e)
                u_ = draw((F, H), t + 9 + 3 * e)
                gus.append(interleave_gate_up(g_, u_))
                downs.append(draw((H, F), t + 10 + 3 * e))
                del g_, u_
            L.ex_wgu = torch.stack(gus)
            L.ex_wdown = torch.stack(downs)
        else:
            F = cfg.ffn
            g_ = shard_rows(draw((F, H), t + 4), tp_rank, tp_world)
            u_ = shard_rows(draw((F, H), t + 5), tp_rank, tp_world)
            L.wgu = interleave_gate_up(g_, u_)
            del g_, u_
            L.wdown = shard_cols(draw((H, F), t + 6), tp_rank, tp_world)
        layers.append(L)
    embed = draw((cfg.vocab, H), 1) if (st.first or (st.last and cfg.tie_embeddings)) else None
    lm_head = None
    if st.last:
        lm_head = embed if cfg.tie_embeddings else draw((cfg.vocab, H), 2)
        if tp_world > 1:
            lm_head = shard_rows(lm_head, tp_rank, tp_world)  # vocabulary-parallel head
    if not st.first:
        embed = None
    dw = DecoderWeights(cfg=cfg, embed=embed, final_norm=ones(H) if st.last else None, lm_head=lm_head,
                        layers=layers, tp_rank=tp_rank, tp_world=tp_world, ep_rank=ep_rank, ep_world=ep_world,
                        stage=stage)
    if cfg.mtp_head:
        eh = draw((H, 2 * H), 3)
        dw.mtp = mtp_input_weights(ones(H), ones(H), eh)
    return fold_scales(dw)


def from_named_tensors(cfg: DecoderConfig, tensors: Dict[str, torch.Tensor], device, tp_rank: int = 0,
                       tp_world: int = 1, dtype=torch.bfloat16, stage: Optional[StageSpec] = None,
                       packed_experts: Optional[dict] = None) -> DecoderWeights:
    """Build device weights from canonical names (``layers.{i}.attn_q`` ... as produced by the family name tables).
    ``packed_experts``: layer index -> ``PackedExperts`` for layers whose routed experts stay as stored (their
    ``experts.*`` tensors are then not read here)."""
    dev = torch.device(device)

    def get(name):
        return tensors[name].to(device=dev, dtype=dtype)

    layers = []
    st = stage or StageSpec.whole(cfg)
    for l in range(st.l0, st.l1):
        p = f"layers.{l}."
        pre = cfg.block in ("pre", "sandwich")
        if cfg.mixer_of(l) == "gdn":
            # one GEMM for every projection of the layer: q | k | v | z | b | a rows
            w_in = torch.cat([get(p + r) for r in ("gdn_q", "gdn_k", "gdn_v", "gdn_z", "gdn_b", "gdn_a")], 0).contiguous()
            f32 = lambda n: tensors[p + n].to(device=dev, dtype=torch.float32).contiguous()
            L = LayerWeights(ln1=get(p + "attn_norm"), ln2=get(p + "ffn_norm"), wqkv=w_in, wo=get(p + "gdn_o"), kind="gdn",
                             gdn={"conv": f32("gdn_conv"), "dt_bias": f32("gdn_dt_bias"), "a_log": f32("gdn_a_log"),
                                  "gate_norm": get(p + "gdn_gate_norm_w")})
        elif cfg.mixer_of(l) == "mamba":
            # one GEMM for z | (x | B | C) | dt; rows padded to a multiple of 8 for the tiled GEMM's output alignment
            w_in = torch.cat([get(p + r) for r in ("ssm_in_z", "ssm_in_x", "ssm_in_dt")], 0)
            pad = (-w_in.shape[0]) % 8
            if pad:
                w_in = torch.cat([w_in, torch.zeros(pad, w_in.shape[1], dtype=dtype, device=dev)], 0)
            f32 = lambda n: tensors[p + n].to(device=dev, dtype=torch.float32).contiguous()
            L = LayerWeights(ln1=get(p + "attn_norm"), ln2=None, wqkv=w_in.contiguous(), wo=get(p + "ssm_o"), kind="mamba",
                             ssm={"conv": f32("ssm_conv"), "conv_bias": f32("ssm_conv_bias") if cfg.ssm_conv_bias else None,
                                  "dt_bias": f32("ssm_dt_bias"), "a_log": f32("ssm_a_log"), "d": f32("ssm_d"),
                                  "gate_norm": get(p + "ssm_gate_norm_w")})
        elif cfg.mixer_of(l) == "none":
            L = LayerWeights(ln1=None, ln2=None, wqkv=None, wo=None, kind="none")
        elif cfg.is_mla:
            m = {"kv_a": get(p + "attn_kv_a"), "kv_a_norm": get(p + "attn_kv_a_norm"), "kv_b": get(p + "attn_kv_b")}
            if cfg.q_lora_rank:
                m.update({"q_a": get(p + "attn_q_a"), "q_a_norm": get(p + "attn_q_a_norm"), "q_b": get(p + "attn_q_b")})
            else:
                m["q"] = get(p + "attn_q")
            if cfg.index_topk:
                # sparse attention indexer: its query heads read the low-rank query, its key and head weights the layer
                # input; the head-weight rows carry the 1/sqrt(heads) factor and are padded to a multiple of 8 rows
                ni = cfg.index_n_heads
                wts = tensors[p + "idx_weights"].to(device=dev, dtype=torch.float32) * (ni ** -0.5)
                pad = (-ni) % 8
                if pad:
                    wts = torch.cat([wts, torch.zeros(pad, wts.shape[1], dtype=torch.float32, device=dev)], 0)
                m.update({"idx_q": get(p + "idx_q"), "idx_k": get(p + "idx_k"), "idx_k_norm": get(p + "idx_k_norm"),
                          "idx_k_norm_bias": get(p + "idx_k_norm_bias"), "idx_w": wts.to(dtype).contiguous()})
            L = LayerWeights(ln1=get(p + "attn_norm"), ln2=get(p + "ffn_norm"), wqkv=m["kv_a"], wo=get(p + "attn_o"), kind="mla", mla=m)
        else:
            wqkv = fuse_qkv(get(p + "attn_q"), get(p + "attn_k"), get(p + "attn_v"), cfg, tp_rank, tp_world)
            wo = shard_cols(get(p + "attn_o"), tp_rank, tp_world)
            L = LayerWeights(ln1=get(p + "attn_norm") if pre else None,
                             ln2=get(p + "ffn_norm") if (pre and cfg.has_ffn(l)) else None, wqkv=wqkv, wo=wo)
            if cfg.attn_gate:
                L.wgate = shard_rows(get(p + "attn_gate"), tp_rank, tp_world)
            if cfg.out_bias:
                L.bo = get(p + "attn_o_bias")
            if cfg.attn_sinks:                   # one sink logit per query head: a rank keeps its heads'
                hq = cfg.n_heads // tp_world
                L.sinks = tensors[p + "attn_sinks"][tp_rank * hq:(tp_rank + 1) * hq].to(device=dev, dtype=torch.float32).contiguous()
        if cfg.block in ("post", "sandwich"):
            L.post1, L.post2 = get(p + "attn_post_norm"), get(p + "ffn_post_norm")
        if cfg.attn_bias:
            L.bqkv = fuse_qkv_bias(get(p + "attn_q_bias"), get(p + "attn_k_bias"), get(p + "attn_v_bias"), cfg, tp_rank, tp_world)
        if cfg.qk_norm and L.kind == "attention":
            L.q_norm, L.k_norm = get(p + "attn_q_norm"), get(p + "attn_k_norm")
            if cfg.qk_norm_wide and tp_world > 1:     # a weight per projection channel: a rank keeps its heads' channels
                L.q_norm = shard_rows(L.q_norm, tp_rank, tp_world)
                L.k_norm = shard_rows(L.k_norm, tp_rank, tp_world)
        if cfg.has_ffn(l) and L.ln2 is None and cfg.block != "post":
            L.ln2 = get(p + "ffn_norm")
        if not cfg.has_ffn(l):
            pass
        elif cfg.moe_layer(l):
            L.router = get(p + "ffn_router")
            if cfg.router_select_bias:
                L.select_bias = tensors[p + "ffn_router_select_bias"].to(device=dev, dtype=torch.float32).contiguous()
            if cfg.router_bias:
                L.router_bias = tensors[p + "ffn_router_bias"].to(device=dev, dtype=torch.float32).contiguous()
            if cfg.expert_bias and not (packed_experts and l in packed_experts):
                b = get(p + "experts_in_bias")                       # [E, 2F]: gate half then up half
                F_ = cfg.moe_ffn
                L.ex_bgu = torch.stack([b[:, :F_], b[:, F_:]], dim=2).reshape(b.shape[0], 2 * F_).contiguous()
                L.ex_bdown = get(p + "experts_out_bias")
            if cfg.shared_width:
                L.sh_wgu = interleave_gate_up(get(p + "shared_gate"), get(p + "shared_up")) if cfg.gated_ffn else get(p + "shared_up")
                L.sh_wdown = get(p + "shared_down")
                if cfg.shared_expert_gate:
                    L.sh_gate = torch.zeros(8, cfg.hidden, dtype=dtype, device=dev)
                    L.sh_gate[0] = get(p + "shared_expert_gate")[0]
            if packed_experts and l in packed_experts:
                L.ex_packed = packed_experts[l]           # the experts stay as stored; biases live on the packed object
                L.ex_bgu = L.ex_bdown = None
            else:
                gus, downs = [], []
                for e in range(cfg.n_experts):
                    gus.append(interleave_gate_up(get(p + f"experts.{e}.gate"), get(p + f"experts.{e}.up")) if cfg.gated_ffn
                               else get(p + f"experts.{e}.up"))
                    downs.append(get(p + f"experts.{e}.down"))
                L.ex_wgu, L.ex_wdown = torch.stack(gus), torch.stack(downs)
        elif cfg.gated_ffn:
            L.wgu = interleave_gate_up(shard_rows(get(p + "ffn_gate"), tp_rank, tp_world),
                                       shard_rows(get(p + "ffn_up"), tp_rank, tp_world))
            L.wdown = shard_cols(get(p + "ffn_down"), tp_rank, tp_world)
        else:                                   # down(act(up(x))): no gate
            L.wgu = shard_rows(get(p + "ffn_up"), tp_rank, tp_world)
            L.wdown = shard_cols(get(p + "ffn_down"), tp_rank, tp_world)
            if cfg.mlp_bias:
                L.bgu, L.bdown = shard_rows(get(p + "ffn_up_bias"), tp_rank, tp_world), get(p + "ffn_down_bias")
        if cfg.norm_kind == "layer" and cfg.norm_bias:
            L.ln1_b, L.ln2_b = get(p + "attn_norm_bias"), get(p + "ffn_norm_bias")
        layers.append(L)
    tied = cfg.tie_embeddings or "lm_head" not in tensors
    embed = get("embed") if (st.first or (st.last and tied)) else None
    lm_head = None
    if st.last:
        lm_head = embed if tied else get("lm_head")
        if tp_world > 1:
            lm_head = shard_rows(lm_head, tp_rank, tp_world)
    if not st.first:
        embed = None
    dw = DecoderWeights(cfg=cfg, embed=embed, final_norm=get("final_norm") if st.last else None,
                        lm_head=lm_head, layers=layers, tp_rank=tp_rank, tp_world=tp_world, stage=stage)
    if cfg.mtp_head:
        dw.mtp = mtp_input_weights(get("mtp.enorm"), get("mtp.hnorm"), get("mtp.eh_proj"))
    if cfg.norm_kind == "layer" and cfg.norm_bias and st.last:
        dw.final_norm_b = get("final_norm_bias")
    if cfg.embed_norm and st.first:
        dw.embed_norm = get("embed_norm")
        dw.embed_norm_b = get("embed_norm_bias") if cfg.norm_bias else None
    return fold_scales(dw)


def random_quant_weights(cfg: DecoderConfig, device, proj_format: str = "Q4_K", embed_format: str = "Q8_0", seed: int = 0,
                         std: float = 0.02, tp_rank: int = 0, tp_world: int = 1) -> DecoderWeights:
    """Weight-only block-quantised model: the random bf16 model of :func:`random_weights`, each projection encoded
    on the device in ``proj_format`` and the token / output embeddings in ``embed_format``; norms stay bf16.

    Rank shares are cut before encoding; every cut falls on a block boundary (rows for q/k/v/gate/up, multiples of
    the 256-value super-block along ``in`` for o/down), so a share equals the same slice of the whole packed tensor.
    """
    from ..ops.cuda_ops import QuantWeight
    from ..quant.torch_quant import ENCODERS
    if cfg.is_moe:
        raise ValueError("quantised expert weights are not built")
    dense = random_weights(cfg, device, seed=seed, std=std, tp_rank=tp_rank, tp_world=tp_world)

    def enc(t: torch.Tensor, fmt: str) -> "QuantWeight":
        rows, cols = t.shape
        parts = [ENCODERS[fmt](t[r:r + 16384]) for r in range(0, rows, 16384)]   # bounded fp32 temporaries
        return QuantWeight(fmt, torch.cat(parts).reshape(-1), rows, cols)

    for L in dense.layers:
        for role in ("wqkv", "wo", "wgu", "wdown"):
            setattr(L, role, enc(getattr(L, role), proj_format))
    tied = dense.lm_head is dense.embed
    dense.embed = enc(dense.embed, embed_format)
    dense.lm_head = dense.embed if tied else enc(dense.lm_head, embed_format)
    return dense
