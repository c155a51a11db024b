"""GLM-5.3-Flash: hyper-connection streams, Kimi delta attention and latent attention under a pooled indexer, each
against a token-by-token restatement in f64 written from the definitions; the whole stack in chunks and decode steps;
a checkpoint directory in the family's own tensor names through the registry, the loader and the driver; the
multi-token-prediction layer as a draft."""
import json

import numpy as np
import pytest

from poot_b200.models.glm53 import Glm53Config, Glm53Model
from poot_b200.models.model import StepSpec
from poot_b200.oracle.runner import OracleSession, random_weights_f32


def _cfg(**kw):
    base = dict(name="glm53_flash", family="glm53_flash", n_layers=4, hidden=16, n_heads=2, n_kv_heads=2, head_dim=6, ffn=24,
                vocab=48, max_position=64, pos="none", layer_kinds=["kda", "dsa", "kda", "dsa"],
                ffn_kinds=["dense", "sparse", "sparse", "sparse"], kda_heads=2, kda_head_dim=8, kda_conv=4, kda_lower_bound=-5.0,
                hc_mult=2, hc_eps=1e-6, hc_iters=3, q_lora_rank=8, kv_lora_rank=8, qk_nope_dim=6, v_head_dim=6, index_n_heads=2,
                index_head_dim=8, index_topk=4, index_kpool=2, n_experts=6, top_k=2, moe_ffn=12, n_shared_experts=1,
                routed_scale=2.5, router="sigmoid", router_select_bias=True, swiglu_limit=0.5, mtp_layers=1)
    base.update(kw)
    return Glm53Config(**base)


def _weights(model, seed=0):
    w = random_weights_f32(model, seed=seed, std=0.5)
    rng = np.random.default_rng(seed + 100)
    for n in w:
        if n.endswith(("_scale",)) or "norm" in n and not n.endswith("_bias"):
            w[n] = (1.0 + 0.2 * rng.standard_normal(w[n].shape)).astype(np.float32)
        elif n.endswith(("_base", "_bias", "select_bias")):
            w[n] = (0.2 * rng.standard_normal(w[n].shape)).astype(np.float32)
    return w


# ---- the definitions, token by token, in f64 ------------------------------------------------------------------------
def _sig(x):
    return 1.0 / (1.0 + np.exp(-x))


def _rms(x, w, eps):
    return x / np.sqrt((x * x).mean() + eps) * w


class Restated:
    """One sequence through the stack one token at a time; every cache is a Python list of what a position stored."""

    def __init__(self, cfg, w):
        self.c, self.w = cfg, {k: np.asarray(v, np.float64) for k, v in w.items()}
        self.pos = 0
        self.kda = {}                # layer -> (window rows, state)
        self.dsa = {}                # layer -> dict of per-position lists

    def W(self, n):
        return self.w[n]

    def site(self, xs, p, site):
        c = self.c
        S = c.hc_mult
        flat = np.concatenate(xs)
        mix = self.W(p + f"hc_{site}_fn") @ (flat / np.sqrt((flat * flat).mean() + c.norm_eps))
        base, scale = self.W(p + f"hc_{site}_base"), self.W(p + f"hc_{site}_scale")
        pre = _sig(mix[:S] * scale[0] + base[:S]) + c.hc_eps
        post = 2.0 * _sig(mix[S:2 * S] * scale[1] + base[S:2 * S])
        logits = mix[2 * S:].reshape(S, S) * scale[2] + base[2 * S:].reshape(S, S)
        e = np.exp(logits - logits.max(1, keepdims=True))
        comb = e / e.sum(1, keepdims=True) + c.hc_eps
        comb = comb / (comb.sum(0, keepdims=True) + c.hc_eps)
        for _ in range(1, c.hc_iters):
            comb = comb / (comb.sum(1, keepdims=True) + c.hc_eps)
            comb = comb / (comb.sum(0, keepdims=True) + c.hc_eps)
        return sum(pre[s] * xs[s] for s in range(S)), post, comb

    def place(self, xs, post, comb, out):
        S = self.c.hc_mult
        return [post[s] * out + sum(comb[j, s] * xs[j] for j in range(S)) for s in range(S)]

    def kda_block(self, l, x):
        c, p = self.c, f"layers.{l}."
        h, d, K = c.kda_heads, c.kda_head_dim, c.kda_conv
        C = h * d
        win, S = self.kda.get(l, ([np.zeros(3 * C)] * (K - 1), np.zeros((h, d, d))))
        raw = np.concatenate([self.W(p + "kda_q") @ x, self.W(p + "kda_k") @ x, self.W(p + "kda_v") @ x])
        taps = np.concatenate([self.W(p + "kda_conv_q"), self.W(p + "kda_conv_k"), self.W(p + "kda_conv_v")], 0)
        seen = win + [raw]                                             # oldest first, K rows
        y = sum(taps[:, k] * seen[k] for k in range(K))
        y = y * _sig(y)
        q, k, v = (y[i * C:(i + 1) * C].reshape(h, d) for i in range(3))
        q = q / np.sqrt((q * q).sum(1, keepdims=True) + 1e-6) / np.sqrt(d)
        k = k / np.sqrt((k * k).sum(1, keepdims=True) + 1e-6)
        f = (self.W(p + "kda_f_b") @ (self.W(p + "kda_f_a") @ x) + self.W(p + "kda_dt_bias")).reshape(h, d)
        g = c.kda_lower_bound * _sig(np.exp(self.W(p + "kda_a_log"))[:, None] * f)
        beta = _sig(self.W(p + "kda_b") @ x)
        S = S.copy()
        o = np.zeros((h, d))
        for i in range(h):
            S[i] = np.exp(g[i])[:, None] * S[i]
            delta = beta[i] * (v[i] - k[i] @ S[i])
            S[i] = S[i] + np.outer(k[i], delta)
            o[i] = q[i] @ S[i]
        self.kda[l] = (seen[1:], S)
        gate = _sig(self.W(p + "kda_g_b") @ (self.W(p + "kda_g_a") @ x)).reshape(h, d)
        o = np.stack([_rms(o[i], self.W(p + "kda_o_norm"), c.norm_eps) for i in range(h)]) * gate
        return self.W(p + "kda_o") @ o.reshape(-1)

    def kept_positions(self, l, x, qr):
        """Positions the query at ``self.pos`` attends: the best complete pools and the tail after the last one."""
        c, p = self.c, f"layers.{l}."
        st = self.dsa[l]
        ni, di, pool = c.index_n_heads, c.index_head_dim, c.index_kpool
        complete = (self.pos + 1) // pool
        tail = list(range(complete * pool, self.pos + 1))
        if complete == 0:
            return tail
        q = (self.W(p + "idx_q") @ qr).reshape(ni, di)
        hw = self.W(p + "idx_weights") @ x / np.sqrt(ni)
        bias = self.W(p + "idx_pool_bias")
        scores = []
        for j in range(complete):
            keys = np.stack(st["key"][j * pool:(j + 1) * pool])                     # [pool, di]
            gates = np.stack(st["gate"][j * pool:(j + 1) * pool]) + bias
            e = np.exp(gates - gates.max(0, keepdims=True))
            pooled = (e / e.sum(0, keepdims=True) * keys).sum(0)
            scores.append(float((hw * np.maximum(q @ pooled, 0.0) / np.sqrt(di)).sum()))
        order = sorted(range(complete), key=lambda j: (-np.float32(scores[j]), j))
        kept = sorted(order[:c.index_topk // pool])
        return [j * pool + i for j in kept for i in range(pool)] + tail

    def dsa_block(self, l, x):
        c, p = self.c, f"layers.{l}."
        nh, qk, vd = c.n_heads, c.qk_nope_dim, c.v_head_dim
        st = self.dsa.setdefault(l, {"c": [], "key": [], "gate": []})
        qr = _rms(self.W(p + "attn_q_a") @ x, self.W(p + "attn_q_a_norm"), c.norm_eps)
        q = (self.W(p + "attn_q_b") @ qr).reshape(nh, qk)
        st["c"].append(_rms(self.W(p + "attn_kv_a") @ x, self.W(p + "attn_kv_a_norm"), c.norm_eps))
        raw = self.W(p + "idx_k") @ x
        cen = raw - raw.mean()
        st["key"].append(cen / np.sqrt((cen * cen).mean() + 1e-6) * self.W(p + "idx_k_norm") + self.W(p + "idx_k_norm_bias"))
        st["gate"].append(self.W(p + "idx_pool_gate") @ x)
        keep = self.kept_positions(l, x, qr)
        kv = np.stack([(self.W(p + "attn_kv_b") @ st["c"][s]).reshape(nh, qk + vd) for s in keep])    # [n, nh, qk + vd]
        out = np.zeros((nh, vd))
        for h in range(nh):
            sc = kv[:, h, :qk] @ q[h] / np.sqrt(qk)
            e = np.exp(sc - sc.max())
            out[h] = (e / e.sum()) @ kv[:, h, qk:]
        return self.W(p + "attn_o") @ out.reshape(-1), keep

    def glu(self, g, u):
        lim = self.c.swiglu_limit
        g = np.minimum(g, lim)
        return g * _sig(g) * np.clip(u, -lim, lim)

    def ffn_block(self, l, x):
        c, p = self.c, f"layers.{l}."
        if c.ffn_kind(l) == "dense":
            return self.W(p + "ffn_down") @ self.glu(self.W(p + "ffn_gate") @ x, self.W(p + "ffn_up") @ x)
        scores = _sig(self.W(p + "ffn_router") @ x)
        choice = scores + self.W(p + "ffn_router_select_bias")
        sel = sorted(range(c.n_experts), key=lambda e: (-np.float32(choice[e]), e))[:c.top_k]
        gates = scores[sel]
        if c.norm_topk_prob:
            gates = gates / (gates.sum() + 1e-20)
        out = np.zeros(c.hidden)
        F = c.moe_ffn
        for gt, e in zip(gates * c.routed_scale, sel):
            gu = self.W(p + "experts_in")[e] @ x
            out += gt * (self.W(p + "experts_out")[e] @ self.glu(gu[:F], gu[F:]))
        return out + self.W(p + "shared_down") @ self.glu(self.W(p + "shared_gate") @ x, self.W(p + "shared_up") @ x)

    def token(self, tok, carry=None):
        """Logits and the closing-norm hidden state of one more token."""
        c = self.c
        h = self.W("embed")[tok]
        if c.mtp_head:
            e = np.zeros_like(h) if self.pos == 0 else h
            h = self.W("mtp.eh_proj") @ np.concatenate([_rms(e, self.W("mtp.enorm"), c.norm_eps), _rms(carry, self.W("mtp.hnorm"), c.norm_eps)])
        mixer = lambda l, x: self.kda_block(l, x) if c.mixer_of(l) == "kda" else self.dsa_block(l, x)[0]
        if c.hyper:
            xs = [h.copy() for _ in range(c.hc_mult)]
            for l in range(c.n_layers):
                p = f"layers.{l}."
                for site, block, nrm in (("attn", mixer, "attn_norm"), ("ffn", self.ffn_block, "ffn_norm")):
                    x, post, comb = self.site(xs, p, site)
                    xs = self.place(xs, post, comb, block(l, _rms(x, self.W(p + nrm), c.norm_eps)))
            h = sum(xs) / c.hc_mult
        else:
            for l in range(c.n_layers):
                p = f"layers.{l}."
                h = h + mixer(l, _rms(h, self.W(p + "attn_norm"), c.norm_eps))
                h = h + self.ffn_block(l, _rms(h, self.W(p + "ffn_norm"), c.norm_eps))
        x = _rms(h, self.W("final_norm"), c.norm_eps)
        self.pos += 1
        return (self.W("embed") if c.tie_embeddings else self.W("lm_head")) @ x, x


# ---- the traced stack against the restatement ---------------------------------------------------------------------------
@pytest.mark.parametrize("variant", ["fixture", "finetune"])
def test_traced_stack_equals_the_token_by_token_restatement(variant):
    """Prefill in two chunks, then decode steps: every position's logits equal the f64 restatement.  The fixture keeps 2
    of up to 8 complete pools of 2 positions, so most positions are outside some query's attention; the fine-tune has
    three layers in another order, three heads, pools of 3 and fewer experts."""
    cfg = _cfg() if variant == "fixture" else _cfg(
        n_layers=3, layer_kinds=["kda", "dsa", "kda"], ffn_kinds=["dense", "dense", "sparse"], n_experts=4, top_k=3, n_heads=3,
        n_kv_heads=3, kda_heads=3, index_kpool=3, index_topk=6, mtp_layers=0, hc_mult=3, hc_iters=2)
    m = Glm53Model(cfg)
    w = _weights(m, seed=3)
    toks = np.random.default_rng(5).integers(0, cfg.vocab, 17)
    ref = Restated(cfg, w)
    want = np.stack([ref.token(int(t))[0] for t in toks])
    s = OracleSession(m, w, rows=1, capacity=32, paged=True, logit_rows="all")
    got = np.concatenate([s.step(toks[None, :7]), s.step(toks[None, 7:12])] + [s.step(toks[None, t:t + 1]) for t in range(12, 17)])
    assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())
    # the selection is live: some query leaves visible positions out
    dsa_layer = cfg.layer_kinds.index("dsa")
    probe = Restated(cfg, w)
    dropped = 0
    for t in toks:
        probe.token(int(t))
    x = np.random.default_rng(1).standard_normal(cfg.hidden)
    probe.pos -= 1
    keep = probe.kept_positions(dsa_layer, x, np.random.default_rng(2).standard_normal(cfg.q_lora_rank))
    assert len(keep) < len(toks)


def test_one_shot_prefill_equals_chunks_and_steps_bitwise_close():
    cfg = _cfg()
    m = Glm53Model(cfg)
    w = _weights(m, seed=1)
    toks = np.random.default_rng(2).integers(0, cfg.vocab, (1, 13))
    full = OracleSession(m, w, rows=1, capacity=32, paged=True).step(toks)
    s = OracleSession(m, w, rows=1, capacity=32, paged=True)
    s.step(toks[:, :6])
    s.step(toks[:, 6:10])
    for t in range(10, 13):
        last = s.step(toks[:, t:t + 1])
    assert np.abs(full - last).max() <= 1e-5


def test_hyper_connection_site_is_near_doubly_stochastic_and_places_the_output_on_every_stream():
    from poot_b200.ir.builder import Builder
    from poot_b200.models import components as C
    from poot_b200.oracle.eval import eval_graph
    from poot_b200.tensor import DType
    L, S, H = 5, 3, 4
    b = Builder()
    xs = b.slot("xs", (L, S, H), DType.F32, "activation")
    fn = b.slot("fn", ((2 + S) * S, S * H), DType.F32, "activation")
    base = b.slot("base", ((2 + S) * S,), DType.F32, "activation")
    scale = b.slot("scale", (3,), DType.F32, "activation")
    out = b.slot("out", (L, H), DType.F32, "activation")
    x, post, comb = C.mhc_pre(b, xs, fn, base, scale, 1e-5, 1e-6, 8)
    b.output(x, "x"); b.output(post, "post"); b.output(comb, "comb"); b.output(C.mhc_post(b, post, comb, out, xs), "next")
    rng = np.random.default_rng(0)
    feed = {"xs": rng.standard_normal((L, S, H)), "fn": rng.standard_normal(((2 + S) * S, S * H)), "base": rng.standard_normal((2 + S) * S) * 0.3,
            "scale": np.array([0.9, 1.1, 1.3]), "out": rng.standard_normal((L, H))}
    feed = {k: v.astype(np.float32) for k, v in feed.items()}
    r = eval_graph(b.finish(), feed).outputs
    assert np.allclose(r["comb"].sum(1), 1.0, atol=1e-4) and np.allclose(r["comb"].sum(2), 1.0, atol=0.1)     # ends on the column step
    assert (r["post"] > 0).all() and (r["post"] < 2).all()
    want = r["post"][:, :, None] * feed["out"][:, None, :] + np.einsum("ljs,ljh->lsh", r["comb"], feed["xs"])
    assert np.allclose(r["next"], want, atol=1e-5)


def test_delta_rule_scan_with_a_decay_per_key_channel():
    """The scan equation's log decay may be one value per head and token or one per key channel; the second decays row
    ``i`` of the state by ``exp(g[i])``."""
    from poot_b200.ir.builder import Builder
    from poot_b200.ir.graph import GraphError
    from poot_b200.oracle.eval import eval_graph
    from poot_b200.tensor import DType
    H, T, D = 2, 5, 4
    rng = np.random.default_rng(0)
    feed = {n: rng.standard_normal(s).astype(np.float32) for n, s in
            (("q", (1, H, T, D)), ("k", (1, H, T, D)), ("v", (1, H, T, D)), ("beta", (1, H, T, 1)), ("s", (1, H, D, D)))}
    feed["g"] = -np.abs(rng.standard_normal((1, H, T, D))).astype(np.float32)
    b = Builder()
    ins = {n: b.slot(n, a.shape, DType.F32, "activation") for n, a in feed.items()}
    y, so = b.scan("delta_rule", [ins[n] for n in ("q", "k", "v", "g", "beta", "s")])
    b.output(y, "y"); b.output(so, "s_out")
    r = eval_graph(b.finish(), feed).outputs
    S = feed["s"][0].astype(np.float64)
    for t in range(T):
        for h in range(H):
            S[h] = np.exp(feed["g"][0, h, t].astype(np.float64))[:, None] * S[h]
            d = feed["beta"][0, h, t, 0] * (feed["v"][0, h, t] - feed["k"][0, h, t] @ S[h])
            S[h] = S[h] + np.outer(feed["k"][0, h, t], d)
            assert np.allclose(r["y"][0, h, t], feed["q"][0, h, t] @ S[h], atol=1e-4)
    assert np.allclose(r["s_out"][0], S, atol=1e-4)
    bad = Builder()
    ins = {n: bad.slot(n, a.shape if n != "g" else (1, H, T, 2), DType.F32, "activation") for n, a in feed.items()}
    with pytest.raises(GraphError):
        bad.scan("delta_rule", [ins[n] for n in ("q", "k", "v", "g", "beta", "s")])


# ---- a checkpoint directory in the family's tensor names ------------------------------------------------------------------
def _header():
    text = {"model_type": "glm5_next_text", "vocab_size": 48, "hidden_size": 16, "num_hidden_layers": 4, "num_nextn_predict_layers": 1,
            "layer_types": ["linear_attention", "deepseek_sparse_attention", "linear_attention", "deepseek_sparse_attention"],
            "mlp_layer_types": ["dense", "sparse", "sparse", "sparse"],
            "linear_attn_config": {"num_heads": 2, "head_dim": 8, "short_conv_kernel_size": 4, "gate_lower_bound": -5.0},
            "hc_mult": 2, "hc_eps": 1e-6, "hc_sinkhorn_iters": 3, "rms_norm_eps": 1e-5, "hidden_act": "silu", "max_position_embeddings": 64,
            "eos_token_id": [47], "num_attention_heads": 2, "q_lora_rank": 8, "kv_lora_rank": 8, "qk_nope_head_dim": 6,
            "qk_rope_head_dim": 0, "v_head_dim": 6, "mla_use_nope": True, "index_n_heads": 2, "index_head_dim": 8, "index_topk": 4,
            "index_kpool": 2, "index_kpool_compress": True, "index_kpool_always_select_tail": True,
            "indexer_types": ["full"] * 4, "intermediate_size": 24, "moe_intermediate_size": 12, "n_routed_experts": 6,
            "num_experts_per_tok": 2, "n_shared_experts": 1, "n_group": 1, "topk_group": 1, "routed_scaling_factor": 2.5,
            "norm_topk_prob": True, "scoring_func": "sigmoid", "topk_method": "noaux_tc", "swiglu_limit": 0.5}
    return {"model_type": "glm5_next", "tie_word_embeddings": False, "text_config": text}


CKPT_LAYER = {"attn_norm": "input_layernorm.weight", "ffn_norm": "post_attention_layernorm.weight",
              "kda_q": "self_attn.q_proj.weight", "kda_k": "self_attn.k_proj.weight", "kda_v": "self_attn.v_proj.weight",
              "kda_f_a": "self_attn.f_a_proj.weight", "kda_f_b": "self_attn.f_b_proj.weight", "kda_b": "self_attn.b_proj.weight",
              "kda_g_a": "self_attn.g_a_proj.weight", "kda_g_b": "self_attn.g_b_proj.weight", "kda_a_log": "self_attn.A_log",
              "kda_dt_bias": "self_attn.dt_bias", "kda_o_norm": "self_attn.o_norm.weight", "kda_o": "self_attn.o_proj.weight",
              "attn_q_a": "self_attn.q_a_proj.weight", "attn_q_a_norm": "self_attn.q_a_layernorm.weight",
              "attn_q_b": "self_attn.q_b_proj.weight", "attn_kv_a": "self_attn.kv_a_proj_with_mqa.weight",
              "attn_kv_a_norm": "self_attn.kv_a_layernorm.weight", "attn_kv_b": "self_attn.kv_b_proj.weight",
              "attn_o": "self_attn.o_proj.weight", "idx_q": "self_attn.indexer.wq_b.weight", "idx_k": "self_attn.indexer.wk.weight",
              "idx_weights": "self_attn.indexer.weights_proj.weight", "idx_k_norm": "self_attn.indexer.k_norm.weight",
              "idx_k_norm_bias": "self_attn.indexer.k_norm.bias", "idx_pool_gate": "self_attn.indexer.index_kpool_compress_gate",
              "idx_pool_bias": "self_attn.indexer.index_kpool_compress_ape", "ffn_gate": "mlp.gate_proj.weight",
              "ffn_up": "mlp.up_proj.weight", "ffn_down": "mlp.down_proj.weight", "ffn_router": "mlp.gate.weight",
              "ffn_router_select_bias": "mlp.gate.e_score_correction_bias", "shared_gate": "mlp.shared_experts.gate_proj.weight",
              "shared_up": "mlp.shared_experts.up_proj.weight", "shared_down": "mlp.shared_experts.down_proj.weight"}


def _write_checkpoint(path, w, mw, cfg):
    """``w``: the stack's weights by canonical name, ``mw``: the multi-token-prediction layer's as a one-layer model."""
    import torch
    from safetensors.torch import save_file
    out = {"model.language_model.embed_tokens.weight": w["embed"], "model.language_model.norm.weight": w["final_norm"],
           "lm_head.weight": w["lm_head"]}

    def layer(l_file, l_src, src):
        pre, p = f"model.language_model.layers.{l_file}.", f"layers.{l_src}."
        for n, a in src.items():
            if not n.startswith(p):
                continue
            role = n[len(p):]
            if role.startswith("hc_"):
                out[pre + role] = a
            elif role.startswith("kda_conv_"):
                out[pre + f"self_attn.{role[-1]}_conv1d.weight"] = a[:, None, :]
            elif role == "experts_in":
                F = a.shape[1] // 2
                for e in range(a.shape[0]):
                    out[pre + f"mlp.experts.{e}.gate_proj.weight"], out[pre + f"mlp.experts.{e}.up_proj.weight"] = a[e, :F], a[e, F:]
            elif role == "experts_out":
                for e in range(a.shape[0]):
                    out[pre + f"mlp.experts.{e}.down_proj.weight"] = a[e]
            else:
                out[pre + CKPT_LAYER[role]] = a
    for l in range(cfg.n_layers):
        layer(l, l, w)
    if mw is not None:
        layer(cfg.n_layers, 0, mw)
        pre = f"model.language_model.layers.{cfg.n_layers}."
        out.update({pre + "eh_proj.weight": mw["mtp.eh_proj"], pre + "enorm.weight": mw["mtp.enorm"], pre + "hnorm.weight": mw["mtp.hnorm"],
                    pre + "shared_head.norm.weight": mw["final_norm"]})
    path.mkdir(parents=True, exist_ok=True)
    save_file({k: torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32)) for k, v in out.items()}, str(path / "model.safetensors"),
              metadata={"format": "pt"})
    (path / "config.json").write_text(json.dumps(_header()))


def test_checkpoint_in_the_family_names_loads_generates_and_drafts(tmp_path):
    from poot_b200.driver.handle import ModelHandle
    from poot_b200.llm import LLM
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.models.registry import Registry
    model = Registry.builtin().resolve_hf(_header())
    assert isinstance(model, Glm53Model) and model.cfg.layer_kinds == ["kda", "dsa", "kda", "dsa"] and model.cfg.is_recurrent
    assert model.cfg.index_topk // model.cfg.index_kpool == 2 and model.cfg.swiglu_limit == 0.5 and model.cfg.mtp_layers == 1
    w = _weights(model, seed=7)
    mtp = model.mtp_model()
    assert mtp.cfg.layer_kinds == ["dsa"] and not mtp.cfg.hyper and mtp.cfg.ffn_kinds == ["sparse"]
    mw = _weights(mtp, seed=8)
    _write_checkpoint(tmp_path / "ckpt", w, mw, model.cfg)
    handle = ModelHandle.load(str(tmp_path / "ckpt"))
    got = handle.oracle_weights()
    assert sorted(got) == sorted(w) and all(np.array_equal(got[n], w[n]) for n in w)
    assert handle.has_mtp
    gm = handle.mtp_oracle_weights()
    shared = {"embed": w["embed"], "lm_head": w["lm_head"]}
    assert all(np.array_equal(gm[n], shared.get(n, mw[n])) for n in mtp.weight_shapes())
    # generation through the driver equals the restatement's greedy continuation
    prompt = [int(t) for t in np.random.default_rng(11).integers(0, 47, 21)]       # a chunk of 16, then 5
    ref = Restated(model.cfg, w)
    for t in prompt:
        logits, _ = ref.token(t)
    want = []
    for _ in range(8):
        want.append(int(np.argmax(logits)))
        logits, _ = ref.token(want[-1])
    plain = LLM.oracle(str(tmp_path / "ckpt"), rows=2, max_seq=48, num_blocks=16, prefill_chunk=16)
    p = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    assert plain.generate_tokens(prompt, p) == want
    drafted = LLM.oracle(str(tmp_path / "ckpt"), rows=2, max_seq=48, num_blocks=16, prefill_chunk=16, draft_mtp=2)
    assert drafted.draft is not None and drafted.generate_tokens(prompt, p) == want


def test_mtp_layer_equals_its_restatement():
    cfg = _cfg()
    mtp = Glm53Model(cfg).mtp_model()
    w = _weights(mtp, seed=4)
    rng = np.random.default_rng(0)
    toks = rng.integers(0, cfg.vocab, 9)
    carry = rng.standard_normal((9, cfg.hidden)).astype(np.float32)
    ref = Restated(mtp.cfg, w)
    want = np.stack([ref.token(int(t), carry[i].astype(np.float64))[0] for i, t in enumerate(toks)])
    from poot_b200.oracle.eval import EvalOptions, eval_graph
    g = mtp.trace(StepSpec(rows=1, tokens=9, capacity=16, logit_rows="all"))
    feed = {"tokens": toks[None].astype(np.int32), "positions": np.arange(9, dtype=np.int32)[None], "carry": carry,
            "read_map": np.arange(16, dtype=np.int32)[None], "write_map": np.arange(9, dtype=np.int32)}
    for i in g.inputs:
        if i.storage == "const":
            feed[i.name] = w[i.name]
        elif i.storage == "state":
            feed[i.name] = np.zeros(g.types[i.value].shape, np.float32)
    got = eval_graph(g, feed, EvalOptions(matmul_precision="exact")).outputs["logits"]
    assert np.abs(got - want).max() <= 2e-4 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("change,words", [
    ({"hidden_act": "gelu"}, "hidden_act"), ({"scoring_func": "softmax"}, "scoring_func"), ({"mla_use_nope": False}, "mla_use_nope"),
    ({"qk_rope_head_dim": 8}, "rotary"), ({"indexer_types": ["full", "shared", "full", "full"]}, "indexer types"),
    ({"index_topk": 5}, "index_topk"), ({"layer_types": ["linear_attention"] * 3}, "layer schedule"),
    ({"linear_attn_config": {"num_heads": 2}}, "linear_attn_config")])
def test_header_values_the_tracer_does_not_implement_are_refused_by_name(change, words):
    from poot_b200.models.registry import Registry, UnsupportedFamily
    h = _header()
    h["text_config"].update(change)
    with pytest.raises(UnsupportedFamily, match=words):
        Registry.builtin().resolve_hf(h)


def test_device_load_names_what_is_missing(tmp_path):
    from poot_b200.models.registry import Registry
    gaps = Registry.builtin().resolve_hf(_header()).cfg.device_gaps()
    assert any("hyper-connection" in g for g in gaps) and any("delta attention" in g for g in gaps)


def test_kda_scan_host_restatement_equals_the_scan_equation_and_is_what_the_planner_names():
    """The device kernel's host restatement (what the GPU test compares the kernel with) against the oracle's scan
    equation over the same rows; the planner gives a delta rule with a per-channel decay the KDA kernel."""
    import torch
    from poot_b200.oracle.eval import _scan
    from poot_b200.plan import compile_graph
    from poot_b200.utils import kernel_emulation as emu
    torch.manual_seed(0)
    heads, D, T = 2, 8, 6
    C = heads * D
    qkv, f = (torch.randn(T, 3 * C) * 0.5).to(torch.bfloat16), torch.randn(T, C).to(torch.bfloat16)
    bm = torch.randn(T, heads).to(torch.bfloat16)
    dt, al = torch.randn(C) * 0.3, torch.randn(heads) * 0.3
    st, out = torch.zeros(1, heads, D, D), torch.zeros(T, C, dtype=torch.bfloat16)
    emu.kda_scan(qkv, f, bm, 0, dt, al, -5.0, st, torch.tensor([[0, T, 0, 0]], dtype=torch.int32), out, heads, D)
    x = qkv.float().numpy()
    unit = lambda t: t / np.sqrt((t * t).sum(-1, keepdims=True) + 1e-6)
    by_head = lambda a: np.ascontiguousarray(a.reshape(T, heads, D).transpose(1, 0, 2)[None], dtype=np.float32)
    q = by_head(unit(x[:, :C].reshape(T, heads, D)) * D ** -0.5)
    k, v = by_head(unit(x[:, C:2 * C].reshape(T, heads, D))), by_head(x[:, 2 * C:])
    gate = _sig(np.exp(al.numpy())[None, :, None] * (f.float().numpy() + dt.numpy()).reshape(T, heads, D))
    g = by_head(-5.0 * gate)
    beta = np.ascontiguousarray(_sig(bm.float().numpy()).T[None, :, :, None], dtype=np.float32)
    r = _scan("delta_rule", [q, k, v, g, beta, np.zeros((1, heads, D, D), np.float32)])
    assert np.abs(r[0, :, :T].transpose(1, 0, 2).reshape(T, C) - out.float().numpy()).max() <= 4e-3       # bf16 output rows
    assert np.abs(r[0, :, T:] - st[0].numpy()).max() <= 1e-5
    prog = compile_graph(Glm53Model(_cfg()).trace(StepSpec(rows=1, tokens=3, capacity=16)))
    kernels = [k_ for p in prog.plans if p.kind == "dispatch" for k_ in p.kernels]
    assert kernels.count("poot_kda_scan") == 2 and "poot_gdn_scan" not in kernels
