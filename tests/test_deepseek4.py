"""DeepSeek-V4: the three attention layer kinds (window, heavily compressed, compressed sparse), the shared key-value
head with output de-rotation, sinks, the grouped output projection and the hash / score routed experts against a
token-by-token restatement in f64 written from the definitions; a checkpoint directory in the family's tensor names."""
import json

import numpy as np
import pytest

from poot_b200.models.deepseek4 import DeepseekV4Config, DeepseekV4Model
from poot_b200.oracle.runner import OracleSession, random_weights_f32
from tests.test_glm53 import Restated, _rms, _sig


def _cfg(**kw):
    base = dict(name="deepseek4", family="deepseek4", n_layers=3, hidden=16, n_heads=4, n_kv_heads=1, head_dim=8, ffn=0, vocab=40,
                max_position=64, attn_kinds=["sliding", "csa", "hca"], csa_rate=2, hca_rate=4, sliding_window=5, qk_rope_dim=4,
                q_lora_rank=8, o_groups=2, o_lora_rank=6, index_n_heads=2, index_head_dim=6, index_topk=2, hc_mult=2, hc_iters=3,
                n_experts=6, top_k=2, moe_ffn=12, n_shared_experts=1, routed_scale=1.5, router="sqrtsoftplus", swiglu_limit=0.7,
                hash_layers=1, rope_theta=10000.0, compress_rope_theta=160000.0, norm_eps=1e-6)
    base.update(kw)
    return DeepseekV4Config(**base)


def _weights(model, seed=0):
    cfg = model.cfg
    w = random_weights_f32(model, seed=seed, std=0.5)
    rng = np.random.default_rng(seed + 50)
    for n in w:
        if n.endswith("_scale") or "norm" in n:
            w[n] = (1.0 + 0.2 * rng.standard_normal(w[n].shape)).astype(np.float32)
        elif n.endswith(("_base", "_bias", "select_bias", "sinks")):
            w[n] = (0.3 * rng.standard_normal(w[n].shape)).astype(np.float32)
        elif n.endswith("hash_table"):
            w[n] = rng.integers(0, cfg.n_experts, w[n].shape).astype(np.int32)
    return w


def _turn(v, pos, theta, rot, inverse=False):
    """Interleaved rotary on the trailing ``rot`` channels of ``v[..., D]`` at position ``pos``."""
    out = np.array(v, np.float64)
    D = out.shape[-1]
    for i in range(rot // 2):
        ang = pos * theta ** (-2.0 * i / rot) * (-1.0 if inverse else 1.0)
        a, b = out[..., D - rot + 2 * i].copy(), out[..., D - rot + 2 * i + 1].copy()
        out[..., D - rot + 2 * i] = a * np.cos(ang) - b * np.sin(ang)
        out[..., D - rot + 2 * i + 1] = a * np.sin(ang) + b * np.cos(ang)
    return out


class Restated4(Restated):
    def __init__(self, cfg, w):
        super().__init__(cfg, w)
        self.hist = {}              # (layer, name) -> list per position

    def pooled(self, l, tag, j, entry, overlapping, theta):
        """Entry ``j`` of a compressor from the raw histories."""
        c, p = self.c, f"layers.{l}."
        rate = c.rate_of(l)
        kv, gate, bias = self.hist[(l, tag + "kv")], self.hist[(l, tag + "gate")], self.W(p + tag + "_bias")
        span = range(j * rate, (j + 1) * rate)
        if overlapping:
            ks = [kv[s][entry:] for s in span]
            gs = [gate[s][entry:] + bias[s - j * rate, entry:] for s in span]
            if j > 0:
                prev = range((j - 1) * rate, j * rate)
                ks = [kv[s][:entry] for s in prev] + ks
                gs = [gate[s][:entry] + bias[s - (j - 1) * rate, :entry] for s in prev] + gs
        else:
            ks = [kv[s] for s in span]
            gs = [gate[s] + bias[s - j * rate] for s in span]
        ks, gs = np.stack(ks), np.stack(gs)
        e = np.exp(gs - gs.max(0, keepdims=True))
        out = (e / e.sum(0, keepdims=True) * ks).sum(0)
        return _turn(_rms(out, self.W(p + tag + "_norm"), c.norm_eps), j * rate, theta, c.qk_rope_dim)

    def attention(self, l, x):
        c, p = self.c, f"layers.{l}."
        nh, D, rot, kind, rate, pos = c.n_heads, c.head_dim, c.qk_rope_dim, c.kind_of(l), c.rate_of(l), self.pos
        theta = c.rope_theta if kind == "sliding" else c.compress_rope_theta
        q_res = _rms(self.W(p + "attn_q_a") @ x, self.W(p + "attn_q_a_norm"), c.norm_eps)
        q = (self.W(p + "attn_q_b") @ q_res).reshape(nh, D)
        q = _turn(q / np.sqrt((q * q).mean(1, keepdims=True) + c.norm_eps), pos, theta, rot)
        self.hist.setdefault((l, "kv"), []).append(_turn(_rms(self.W(p + "attn_kv") @ x, self.W(p + "attn_kv_norm"), c.norm_eps), pos, theta, rot))
        keys = [self.hist[(l, "kv")][s] for s in range(max(0, pos - c.sliding_window + 1), pos + 1)]
        self.kept = None
        if kind != "sliding":
            for tag in ("cmp",) + (("idx_cmp",) if kind == "csa" else ()):
                self.hist.setdefault((l, tag + "kv"), []).append(self.W(p + tag + "_kv") @ x)
                self.hist.setdefault((l, tag + "gate"), []).append(self.W(p + tag + "_gate") @ x)
            n = (pos + 1) // rate                                        # complete windows
            if kind == "hca":
                kept = list(range(n))
            else:
                ni, di = c.index_n_heads, c.index_head_dim
                iq = _turn((self.W(p + "idx_q") @ q_res).reshape(ni, di), pos, theta, rot)
                hw = self.W(p + "idx_weights") @ x / np.sqrt(ni)
                sc = [np.float32((hw * np.maximum(iq @ self.pooled(l, "idx_cmp", j, di, True, theta), 0.0) / np.sqrt(di)).sum()) for j in range(n)]
                kept = [j for j in range(n) if sum(1 for o in sc if o > sc[j]) < c.index_topk]
            self.kept = (n, kept)
            keys = keys + [self.pooled(l, "cmp", j, D, kind == "csa", theta) for j in kept]
        keys = np.stack(keys)
        sinks = self.W(p + "attn_sinks")
        out = np.zeros((nh, D))
        for h in range(nh):
            s = keys @ q[h] / np.sqrt(D)
            m = max(s.max(), sinks[h])
            e = np.exp(s - m)
            out[h] = (e / (e.sum() + np.exp(sinks[h] - m))) @ keys
        flat = _turn(out, pos, theta, rot, inverse=True).reshape(-1)
        G, ipg, r = c.o_groups, c.in_per_group, c.o_lora_rank
        oa = self.W(p + "attn_o_a")
        mixed = np.concatenate([oa[g * r:(g + 1) * r] @ flat[g * ipg:(g + 1) * ipg] for g in range(G)])
        return self.W(p + "attn_o") @ mixed

    def ffn_block(self, l, x, tok=None):
        c, p = self.c, f"layers.{l}."
        logits = self.W(p + "ffn_router") @ x
        scores = np.sqrt(np.logaddexp(0.0, logits))
        if l < c.hash_layers:
            sel = [int(e) for e in self.W(p + "ffn_hash_table")[tok]]
        else:
            choice = scores + self.W(p + "ffn_router_select_bias")
            sel = sorted(range(c.n_experts), key=lambda e: (-np.float32(choice[e]), e))[:c.top_k]
        gates = scores[sel] / scores[sel].sum() * c.routed_scale
        out, F = np.zeros(c.hidden), c.moe_ffn
        for gt, e in zip(gates, sel):
            gu = self.W(p + "experts_in")[e] @ x
            out += gt * (self.W(p + "experts_out")[e] @ self.glu(gu[:F], gu[F:]))
        return out + self.W(p + "shared_down") @ self.glu(self.W(p + "shared_gate") @ x, self.W(p + "shared_up") @ x)

    def token(self, tok, carry=None):
        c = self.c
        S = c.hc_mult
        xs = [self.W("embed")[tok].copy() for _ in range(S)]
        for l in range(c.n_layers):
            p = f"layers.{l}."
            x, post, comb = self.site(xs, p, "attn")
            xs = self.place(xs, post, comb, self.attention(l, _rms(x, self.W(p + "attn_norm"), c.norm_eps)))
            x, post, comb = self.site(xs, p, "ffn")
            xs = self.place(xs, post, comb, self.ffn_block(l, _rms(x, self.W(p + "ffn_norm"), c.norm_eps), tok))
        flat = np.concatenate(xs)
        mix = self.W("hc_head_fn") @ (flat / np.sqrt((flat * flat).mean() + c.norm_eps))
        pre = _sig(mix * self.W("hc_head_scale")[0] + self.W("hc_head_base")) + c.hc_eps
        h = sum(pre[s] * xs[s] for s in range(S))
        x = _rms(h, self.W("final_norm"), c.norm_eps)
        self.pos += 1
        return self.W("lm_head") @ x, x


@pytest.mark.parametrize("variant", ["fixture", "other"])
def test_traced_stack_equals_the_token_by_token_restatement(variant):
    """Two prefill chunks then decode steps, every position's logits.  The fixture has one layer of each kind, windows
    of 2 (sparse, 2 kept) and 4 positions under a local window of 5, and a hash-routed first layer; the other
    configuration orders the kinds differently with other rates, three streams and no hash layer."""
    cfg = _cfg() if variant == "fixture" else _cfg(
        n_layers=4, attn_kinds=["hca", "csa", "sliding", "csa"], csa_rate=3, hca_rate=2, sliding_window=3, index_topk=1, hc_mult=3,
        hc_iters=2, hash_layers=0, o_groups=4, n_heads=4, top_k=3)
    m = DeepseekV4Model(cfg)
    w = _weights(m, seed=2)
    toks = np.random.default_rng(7).integers(0, cfg.vocab, 19)
    ref = Restated4(cfg, w)
    want, dropped = [], 0
    for t in toks:
        want.append(ref.token(int(t))[0])
        if ref.kept is not None and cfg.kind_of(cfg.n_layers - 1) == "csa":
            dropped += ref.kept[0] - len(ref.kept[1])
    want = np.stack(want)
    s = OracleSession(m, w, rows=1, capacity=32, paged=True, logit_rows="all")
    got = np.concatenate([s.step(toks[None, :6]), s.step(toks[None, 6:13])] + [s.step(toks[None, t:t + 1]) for t in range(13, 19)])
    assert np.abs(got - want).max() <= 3e-4 * max(1.0, np.abs(want).max())
    if variant == "other":
        assert dropped > 0            # the selection is live: readable windows were left out


def test_capacity_below_one_window_still_writes_the_histories():
    """A step whose cache is shorter than a window attends the local window only; the compressors' raw histories are
    written all the same, so a later step at a larger capacity reads them."""
    cfg = _cfg(attn_kinds=["hca", "csa", "sliding"], hca_rate=32, csa_rate=32, hash_layers=0)
    m = DeepseekV4Model(cfg)
    from poot_b200.models.model import StepSpec
    g = m.trace(StepSpec(rows=1, tokens=3, capacity=16))
    names = {o.state_of for o in g.outputs if o.role == "state_next"}
    assert {"layers.0.cmp_kv_pool", "layers.0.cmp_gate_pool", "layers.1.idx_cmp_kv_pool", "layers.1.idx_cmp_gate_pool"} <= names
    assert cfg.prefill_granule == 32 and _cfg().prefill_granule == 4


# ---- a checkpoint directory in the release's tensor names ------------------------------------------------------------------
def _header():
    return {"model_type": "deepseek_v4", "vocab_size": 40, "hidden_size": 16, "num_hidden_layers": 3, "num_attention_heads": 4,
            "head_dim": 8, "qk_rope_head_dim": 4, "q_lora_rank": 8, "o_groups": 2, "o_lora_rank": 6, "sliding_window": 5,
            "compress_rates": {"compressed_sparse_attention": 2, "heavily_compressed_attention": 4}, "compress_ratios": [0, 2, 4],
            "index_n_heads": 2, "index_head_dim": 6, "index_topk": 2, "hc_mult": 2, "hc_eps": 1e-6, "hc_sinkhorn_iters": 3,
            "rms_norm_eps": 1e-6, "n_routed_experts": 6, "num_experts_per_tok": 2, "moe_intermediate_size": 12, "n_shared_experts": 1,
            "routed_scaling_factor": 1.5, "scoring_func": "sqrtsoftplus", "swiglu_limit": 0.7, "num_hash_layers": 1,
            "rope_theta": 10000.0, "compress_rope_theta": 160000.0, "max_position_embeddings": 64, "eos_token_id": 39}


def _write_checkpoint(path, w, cfg):
    import torch
    from safetensors.torch import save_file
    from poot_b200.load.hf_map import DEEPSEEK4_LAYER, DEEPSEEK4_TOP
    top = {v: k for k, v in DEEPSEEK4_TOP.items()}
    layer = {v: k for k, v in DEEPSEEK4_LAYER.items()}
    out = {}
    for n, a in w.items():
        if n in top:
            out[top[n]] = a
            continue
        l, role = n.split(".")[1], n.split(".", 2)[2]
        pre = f"layers.{l}."
        if role == "experts_in":
            F = a.shape[1] // 2
            for e in range(a.shape[0]):
                out[pre + f"ffn.experts.{e}.w1.weight"], out[pre + f"ffn.experts.{e}.w3.weight"] = a[e, :F], a[e, F:]
        elif role == "experts_out":
            for e in range(a.shape[0]):
                out[pre + f"ffn.experts.{e}.w2.weight"] = a[e]
        elif role == "ffn_hash_table":
            out[pre + "ffn.gate.tid2eid"] = a
        else:
            out[pre + layer[role]] = a
    path.mkdir(parents=True, exist_ok=True)
    save_file({k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in out.items()}, str(path / "model.safetensors"), metadata={"format": "pt"})
    (path / "config.json").write_text(json.dumps(_header()))


def test_checkpoint_in_the_release_names_loads_and_generates(tmp_path):
    from poot_b200.driver.handle import ModelHandle
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.llm import LLM
    from poot_b200.models.registry import Registry
    model = Registry.builtin().resolve_hf(_header())
    assert isinstance(model, DeepseekV4Model) and model.cfg.attn_kinds == ["sliding", "csa", "hca"] and model.cfg.hash_layers == 1
    assert model.cfg.to_dict() == {**_cfg().to_dict(), "eos_token": 39, "router_select_bias": True, "attn_sinks": True, "pos": "rope"}
    w = _weights(model, seed=5)
    _write_checkpoint(tmp_path / "ckpt", w, model.cfg)
    got = ModelHandle.load(str(tmp_path / "ckpt")).oracle_weights()
    assert sorted(got) == sorted(w) and all(np.array_equal(got[n], w[n].astype(np.float32)) for n in w)
    prompt = [int(t) for t in np.random.default_rng(3).integers(0, 39, 19)]           # a chunk of 16, then 3
    ref = Restated4(model.cfg, w)
    for t in prompt:
        logits, _ = ref.token(t)
    want = []
    for _ in range(7):
        want.append(int(np.argmax(logits)))
        logits, _ = ref.token(want[-1])
    llm = LLM.oracle(str(tmp_path / "ckpt"), rows=2, max_seq=48, num_blocks=16, prefill_chunk=16)
    assert llm.generate_tokens(prompt, SamplingParams(max_tokens=7, temperature=0.0, ignore_eos=True)) == want


@pytest.mark.parametrize("change,words", [
    ({"scoring_func": "sigmoid"}, "scoring_func"), ({"rope_scaling": {"rope_type": "yarn", "factor": 4.0}}, "rope_scaling"),
    ({"qk_rope_head_dim": 16}, "qk_rope_head_dim"), ({"o_groups": 3}, "o_groups"), ({"compress_ratios": [0, 2]}, "compress_ratios"),
    ({"compress_ratios": [0, 3, 4]}, "compress_ratios"), ({"index_head_dim": 2}, "indexer"), ({"num_hash_layers": 9}, "num_hash_layers"),
    ({"compress_rates": {"compressed_sparse_attention": 4, "heavily_compressed_attention": 4}}, "compress_rates")])
def test_header_values_the_tracer_does_not_implement_are_refused_by_name(change, words):
    from poot_b200.models.registry import Registry, UnsupportedFamily
    with pytest.raises(UnsupportedFamily, match=words):
        Registry.builtin().resolve_hf({**_header(), **change})


def test_a_table_with_an_expert_id_out_of_range_is_refused_at_load(tmp_path):
    from poot_b200.driver.handle import ModelHandle
    from poot_b200.load.hf_map import CheckpointLayout
    from poot_b200.models.registry import Registry
    model = Registry.builtin().resolve_hf(_header())
    w = _weights(model, seed=5)
    w["layers.0.ffn_hash_table"] = w["layers.0.ffn_hash_table"].copy()
    w["layers.0.ffn_hash_table"][3, 1] = model.cfg.n_experts
    _write_checkpoint(tmp_path / "bad", w, model.cfg)
    with pytest.raises(CheckpointLayout, match="expert ids"):
        ModelHandle.load(str(tmp_path / "bad"))
