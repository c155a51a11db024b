"""Qwen3.8-Flash-Next: gated hyper-connections, the block indexer over full-attention layers, hashed n-gram embedding
blocks and the sigmoid-gated delta net against a token-by-token restatement in f64 written from the definitions; the
n-gram hash constants; a checkpoint directory in the family's tensor names through the loader and the driver."""
import json

import numpy as np
import pytest

from poot_b200.models.ngram import MASK64, ngram_tables
from poot_b200.models.registry import Registry, UnsupportedFamily
from poot_b200.oracle.runner import OracleSession, random_weights_f32
from tests.test_glm53 import _sig


def _header(**text_over):
    text = {"model_type": "qwen4_exp_text", "vocab_size": 60, "hidden_size": 16, "num_hidden_layers": 4, "num_attention_heads": 2,
            "num_key_value_heads": 1, "head_dim": 8, "partial_rotary_factor": 0.5, "rope_theta": 10000.0, "rms_norm_eps": 1e-6,
            "max_position_embeddings": 64, "layer_types": ["linear_attention", "full_attention", "linear_attention", "full_attention"],
            "linear_num_key_heads": 1, "linear_num_value_heads": 2, "linear_key_head_dim": 8, "linear_value_head_dim": 8,
            "linear_conv_kernel_dim": 3, "output_gate_type": "sigmoid", "num_experts": 4, "num_experts_per_tok": 2,
            "moe_intermediate_size": 8, "shared_expert_intermediate_size": 8, "norm_topk_prob": True, "intermediate_size": 8,
            "hc_count": 2, "hc_lowrank": 4, "indexer_n_heads": 2, "indexer_head_dim": 8, "indexer_budget": 4,
            "indexer_compress_ratio": 2, "indexer_kv_heads": 1, "ple_layer_ids": [1, 3], "ple_embed_dim": 8, "ple_conv_kernel_size": 2,
            "ngram_size": 3, "heads_per_ngram": 2, "ngram_vocab_size_base": 50, "make_ngram_vocab_size_divisible_by": 16, "seed": 7,
            "eos_token_id": 59}
    text.update(text_over)
    return {"model_type": "qwen4_exp", "tie_word_embeddings": False, "text_config": text}


def _weights(model, seed=0):
    w = random_weights_f32(model, seed=seed, std=0.5)
    rng = np.random.default_rng(seed + 9)
    for n in w:
        if "norm" in n:
            w[n] = (1.0 + 0.2 * rng.standard_normal(w[n].shape)).astype(np.float32)
        elif n.endswith(("dt_bias", "a_log")):
            w[n] = (0.3 * rng.standard_normal(w[n].shape)).astype(np.float32)
    return w


def _rms(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


def _rope(v, pos, theta, rot):
    """Half-split rotary on the leading ``rot`` channels."""
    out = np.array(v, np.float64)
    h = rot // 2
    for i in range(h):
        ang = pos * theta ** (-2.0 * i / rot)
        a, b = out[..., i].copy(), out[..., i + h].copy()
        out[..., i], out[..., i + h] = a * np.cos(ang) - b * np.sin(ang), b * np.cos(ang) + a * np.sin(ang)
    return out


class Restated38:
    def __init__(self, cfg, w):
        self.c, self.w = cfg, {k: np.asarray(v, np.float64) for k, v in w.items()}
        self.pos, self.tokens = 0, []
        self.gdn, self.att, self.conv = {}, {}, {}
        self.dropped = 0

    def W(self, n):
        return self.w[n]

    def grouped(self, xs, name):
        c = self.c
        return _rms(xs.reshape(c.hc_count, c.hidden), 1.0, c.norm_eps).reshape(-1) * self.W(name)

    def read(self, xs, stem, inject):
        c = self.c
        S = c.hc_count
        n = self.grouped(xs, stem + "norm")
        d = self.W(stem + "down") @ n / S
        gate = _sig(self.W(stem + "up") @ (d * _sig(d)))
        x_in = (gate * n).reshape(S, c.hidden).mean(0)
        return x_in, (2.0 * _sig(self.W(stem + "inject") @ n / S) if inject else None)

    def write(self, xs, out, wts):
        return xs + (wts[:, None] * out[None, :]).reshape(-1)

    def ngram_ids(self, l):
        c = self.c
        tb = c.ple_tables(l)
        eos = c.eos_token
        hist = [eos, eos] + self.tokens                              # before a sequence: end-of-sequence ids
        s0, s1, s2 = hist[-1], hist[-2], hist[-3]
        if s1 == eos:
            s2 = eos
        m = tb.multipliers
        mix2 = ((s0 * m[0]) & MASK64) ^ ((s1 * m[1]) & MASK64)
        mix = [mix2, mix2 ^ ((s2 * m[2]) & MASK64)] if c.ngram_size == 3 else [mix2]
        return [mix[h // c.heads_per_ngram] % tb.primes[h] + tb.offsets[h] for h in range(len(tb.primes))]

    def ple(self, l, xs):
        c, p = self.c, f"layers.{l}."
        S, H, K, dil = c.hc_count, c.hidden, c.ple_conv, c.ngram_size
        emb = np.concatenate([self.W(p + "ple_table")[i] for i in self.ngram_ids(l)])
        key = self.grouped(self.W(p + "ple_key") @ emb, p + "ple_key_norm").reshape(S, H)
        value = self.W(p + "ple_value") @ emb
        query = self.grouped(xs, p + "ple_query_norm").reshape(S, H)
        g = (key * query).sum(1) / np.sqrt(H)
        gate = _sig(np.sign(g) * np.sqrt(np.maximum(np.abs(g), 1e-6)))
        gated = (gate[:, None] * value[None, :]).reshape(-1)
        n = self.grouped(gated, p + "ple_conv_norm")
        past = self.conv.setdefault(("ple", l), [np.zeros(S * H)] * ((K - 1) * dil))
        seen = past + [n]
        taps = self.W(p + "ple_conv")
        y = sum(taps[:, j] * seen[j * dil] for j in range(K))
        self.conv[("ple", l)] = seen[1:]
        return gated + y * _sig(y)

    def gdn_block(self, l, x):
        c, p = self.c, f"layers.{l}."
        nk, nv, D, K = c.gdn_k_heads, c.gdn_v_heads, c.gdn_head_dim, c.gdn_conv
        raw = np.concatenate([self.W(p + "gdn_q") @ x, self.W(p + "gdn_k") @ x, self.W(p + "gdn_v") @ x])
        past, S = self.gdn.get(l, ([np.zeros(raw.shape[0])] * (K - 1), np.zeros((nv, D, D))))
        seen = past + [raw]
        taps = self.W(p + "gdn_conv")
        y = sum(taps[:, k] * seen[k] for k in range(K))
        y = y * _sig(y)
        q, k, v = y[:nk * D].reshape(nk, D), y[nk * D:2 * nk * D].reshape(nk, D), y[2 * nk * D:].reshape(nv, D)
        unit = lambda t: t / np.sqrt((t * t).sum(1, keepdims=True) + 1e-6)
        q, k = np.repeat(unit(q), nv // nk, 0) / np.sqrt(D), np.repeat(unit(k), nv // nk, 0)
        beta = _sig(self.W(p + "gdn_b") @ x)
        g = -np.exp(self.W(p + "gdn_a_log")) * np.logaddexp(0.0, self.W(p + "gdn_a") @ x + self.W(p + "gdn_dt_bias"))
        S, o = S.copy(), np.zeros((nv, D))
        for h in range(nv):
            S[h] = np.exp(g[h]) * S[h]
            S[h] = S[h] + np.outer(k[h], beta[h] * (v[h] - k[h] @ S[h]))
            o[h] = q[h] @ S[h]
        self.gdn[l] = (seen[1:], S)
        z = (self.W(p + "gdn_z") @ x).reshape(nv, D)
        act = _sig(z) if c.gdn_gate_act == "sigmoid" else z * _sig(z)
        return self.W(p + "gdn_o") @ (_rms(o, self.W(p + "gdn_gate_norm_w"), c.norm_eps) * act).reshape(-1)

    def visible(self, l, x):
        """Positions the query at ``self.pos`` reads in a block-indexed layer."""
        c, p = self.c, f"layers.{l}."
        ni, di, ratio, pos = c.index_n_heads, c.index_head_dim, c.index_ratio, self.pos
        st = self.att[l]
        q = _rope(_rms((self.W(p + "idx_q") @ x).reshape(ni, di), self.W(p + "idx_q_norm"), c.norm_eps), pos, c.rope_theta, c.rot)
        complete = (pos + 1) // ratio
        scores = []
        for j in range(complete):
            kb = _rope(_rms(np.mean(st["raw"][j * ratio:(j + 1) * ratio], 0), self.W(p + "idx_k_norm"), c.norm_eps), j * ratio, c.rope_theta, c.rot)
            scores.append(np.float32(np.maximum(q @ kb, 0.0).sum() / np.sqrt(di)))
        kept = sorted(sorted(range(complete), key=lambda j: (-scores[j], j))[:c.index_budget // ratio])
        self.dropped += complete - len(kept)
        return [j * ratio + i for j in kept for i in range(ratio)] + list(range(complete * ratio, pos + 1))

    def attn_block(self, l, x):
        c, p = self.c, f"layers.{l}."
        nh, nkv, D, pos = c.n_heads, c.n_kv_heads, c.head_dim, self.pos
        st = self.att.setdefault(l, {"k": [], "v": [], "raw": []})
        q = _rope(_rms((self.W(p + "attn_q") @ x).reshape(nh, D), self.W(p + "attn_q_norm"), c.norm_eps), pos, c.rope_theta, c.rot)
        st["k"].append(_rope(_rms((self.W(p + "attn_k") @ x).reshape(nkv, D), self.W(p + "attn_k_norm"), c.norm_eps), pos, c.rope_theta, c.rot))
        st["v"].append((self.W(p + "attn_v") @ x).reshape(nkv, D))
        st["raw"].append(self.W(p + "idx_k") @ x)
        keep = self.visible(l, x)
        out = np.zeros((nh, D))
        for h in range(nh):
            kv = h // (nh // nkv)
            s = np.array([st["k"][t][kv] @ q[h] for t in keep]) / np.sqrt(D)
            e = np.exp(s - s.max())
            out[h] = (e / e.sum()) @ np.stack([st["v"][t][kv] for t in keep])
        return self.W(p + "attn_o") @ (out.reshape(-1) * _sig(self.W(p + "attn_gate") @ x))

    def moe_block(self, l, x):
        c, p = self.c, f"layers.{l}."
        logits = self.W(p + "ffn_router") @ x
        sel = sorted(range(c.n_experts), key=lambda e: (-np.float32(logits[e]), e))[:c.top_k]
        e = np.exp(logits[sel] - logits[sel].max())
        out, F = np.zeros(c.hidden), c.moe_ffn
        glu = lambda g, u: g * _sig(g) * u
        for gt, ex in zip(e / e.sum(), sel):
            gu = self.W(p + "experts_in")[ex] @ x
            out += gt * (self.W(p + "experts_out")[ex] @ glu(gu[:F], gu[F:]))
        shared = self.W(p + "shared_down") @ glu(self.W(p + "shared_gate") @ x, self.W(p + "shared_up") @ x)
        return out + shared * _sig(self.W(p + "shared_expert_gate") @ x)

    def token(self, tok):
        c = self.c
        self.tokens.append(int(tok))
        xs = np.tile(self.W("embed")[tok], c.hc_count)
        for l in range(c.n_layers):
            p = f"layers.{l}."
            if c.ple_tables(l) is not None:
                xs = xs + self.ple(l, xs)
            x_in, wts = self.read(xs, p + "hc_attn_", True)
            xs = self.write(xs, self.gdn_block(l, x_in) if c.mixer_of(l) == "gdn" else self.attn_block(l, x_in), wts)
            x_in, wts = self.read(xs, p + "hc_ffn_", True)
            xs = self.write(xs, self.moe_block(l, x_in), wts)
        self.pos += 1
        return self.W("lm_head") @ self.read(xs, "hc_final_", False)[0]


def test_traced_stack_equals_the_token_by_token_restatement():
    """Two prefill chunks (the second starts inside an indexer block and inside an n-gram) and decode steps: every
    position's logits.  Blocks of 2 with a budget of 2 blocks: most complete blocks are dropped for later queries."""
    model = Registry.builtin().resolve_hf(_header())
    cfg = model.cfg
    assert cfg.hc_count == 2 and cfg.ple_layers == [0, 2] and cfg.index_ratio == 2 and cfg.gdn_gate_act == "sigmoid" and cfg.rot == 4
    w = _weights(model, seed=4)
    toks = np.random.default_rng(3).integers(0, cfg.vocab, 18)
    toks[5] = cfg.eos_token                       # an end-of-sequence id inside the run: it hides the tokens before it from order 3
    ref = Restated38(cfg, w)
    want = np.stack([ref.token(int(t)) for t in toks])
    assert ref.dropped > 0
    s = OracleSession(model, w, rows=1, capacity=32, paged=True, logit_rows="all")
    got = np.concatenate([s.step(toks[None, :5]), s.step(toks[None, 5:12])] + [s.step(toks[None, t:t + 1]) for t in range(12, 18)])
    assert np.abs(got - want).max() <= 3e-4 * max(1.0, np.abs(want).max())


def test_ngram_hash_constants_follow_the_derivation():
    """Consecutive primes from the base, each block skipping those of the blocks before it; slices stack into a table
    padded to the multiple; odd multipliers below ``i64::MAX / vocab`` from SplitMix64 of the seed."""
    a, b = ngram_tables(0, 3, 2, 50, 16, 7, 60), ngram_tables(1, 3, 2, 50, 16, 7, 60)
    assert a.primes == (53, 59, 61, 67) and b.primes == (71, 73, 79, 83)
    assert a.offsets == (0, 53, 112, 173) and a.rows == 240 and b.rows == 320
    assert all(m % 2 == 1 and m * 60 < (1 << 63) for m in a.multipliers + b.multipliers) and a.multipliers != b.multipliers
    assert len(ngram_tables(0, 2, 3, 50, 1, 7, 60).primes) == 3 and len(ngram_tables(0, 2, 3, 50, 1, 7, 60).multipliers) == 2
    with pytest.raises(ValueError):
        ngram_tables(0, 4, 2, 50, 16, 7, 60)


@pytest.mark.parametrize("change,words", [
    ({"attention_bias": True}, "attention_bias"), ({"indexer_kv_heads": 2}, "indexer_kv_heads"), ({"indexer_compress_ratio": 3}, "power of two"),
    ({"indexer_budget": 1}, "budget"), ({"ple_layer_ids": [2]}, "ple_layer_ids"), ({"ple_layer_ids": [1, 1]}, "ple_layer_ids"),
    ({"ngram_size": 4}, "n-gram"), ({"ple_embed_dim": 6}, "n-gram"), ({"output_gate_type": "tanh"}, "output_gate_type"),
    ({"partial_rotary_factor": None}, "partial_rotary_factor"), ({"hc_count": 0}, "hc_count"), ({"layer_types": ["full_attention"]}, "layer_types")])
def test_header_values_the_tracer_does_not_implement_are_refused_by_name(change, words):
    with pytest.raises(UnsupportedFamily, match=words):
        Registry.builtin().resolve_hf(_header(**change))


def _write_checkpoint(path, w, cfg):
    """The family's Hugging Face layout: norm scales stored as offsets from one (the delta-net's gated norm as is), the
    attention query and gate rows interleaved per head in ``q_proj``, ``in_proj_qkv`` fused, the indexer's query and key
    rows in one projection, depthwise conv taps as ``[C, 1, K]``."""
    import torch
    from safetensors.torch import save_file
    pre = "model.language_model."
    out = {pre + "embed_tokens.weight": w["embed"], "lm_head.weight": w["lm_head"]}
    gate = lambda stem, src: {stem + "hc_norm.weight": w[src + "norm"] - 1.0, stem + "input_mix_weight_down.weight": w[src + "down"],
                              stem + "input_mix_weight_up.weight": w[src + "up"],
                              **({stem + "block_inject_weight.weight": w[src + "inject"]} if src + "inject" in w else {})}
    out.update(gate(pre + "hyper_connection_mixer.", "hc_final_"))
    D = cfg.head_dim
    for l in range(cfg.n_layers):
        p, q = f"layers.{l}.", f"{pre}layers.{l}."
        out.update(gate(q + "attn_hyper_connection.", p + "hc_attn_"))
        out.update(gate(q + "mlp_hyper_connection.", p + "hc_ffn_"))
        if cfg.ple_tables(l) is not None:
            out.update({q + "ple.ple_embedding.ngram_embedding.weight": w[p + "ple_table"], q + "ple.key_proj.weight": w[p + "ple_key"],
                        q + "ple.value_proj.weight": w[p + "ple_value"], q + "ple.norm_key.weight": w[p + "ple_key_norm"] - 1.0,
                        q + "ple.norm_query.weight": w[p + "ple_query_norm"] - 1.0, q + "ple.norm_conv.weight": w[p + "ple_conv_norm"] - 1.0,
                        q + "ple.conv1d.weight": w[p + "ple_conv"][:, None, :]})
        if cfg.mixer_of(l) == "gdn":
            out.update({q + "linear_attn.in_proj_qkv.weight": np.concatenate([w[p + "gdn_q"], w[p + "gdn_k"], w[p + "gdn_v"]], 0),
                        q + "linear_attn.in_proj_z.weight": w[p + "gdn_z"], q + "linear_attn.in_proj_b.weight": w[p + "gdn_b"],
                        q + "linear_attn.in_proj_a.weight": w[p + "gdn_a"], q + "linear_attn.dt_bias": w[p + "gdn_dt_bias"],
                        q + "linear_attn.A_log": w[p + "gdn_a_log"], q + "linear_attn.norm.weight": w[p + "gdn_gate_norm_w"],
                        q + "linear_attn.out_proj.weight": w[p + "gdn_o"], q + "linear_attn.conv1d.weight": w[p + "gdn_conv"][:, None, :]})
        else:
            H = w[p + "attn_q"].shape[1]
            fused = np.stack([w[p + "attn_q"].reshape(cfg.n_heads, D, H), w[p + "attn_gate"].reshape(cfg.n_heads, D, H)], 1)
            out.update({q + "self_attn.q_proj.weight": fused.reshape(2 * cfg.n_heads * D, H), q + "self_attn.k_proj.weight": w[p + "attn_k"],
                        q + "self_attn.v_proj.weight": w[p + "attn_v"], q + "self_attn.o_proj.weight": w[p + "attn_o"],
                        q + "self_attn.q_norm.weight": w[p + "attn_q_norm"] - 1.0, q + "self_attn.k_norm.weight": w[p + "attn_k_norm"] - 1.0,
                        q + "self_attn.indexer.index_qk_proj.weight": np.concatenate([w[p + "idx_q"], w[p + "idx_k"]], 0),
                        q + "self_attn.indexer.q_layernorm.weight": w[p + "idx_q_norm"] - 1.0,
                        q + "self_attn.indexer.k_layernorm.weight": w[p + "idx_k_norm"] - 1.0})
        F = cfg.moe_ffn
        out.update({q + "mlp.gate.weight": w[p + "ffn_router"], q + "mlp.shared_expert.gate_proj.weight": w[p + "shared_gate"],
                    q + "mlp.shared_expert.up_proj.weight": w[p + "shared_up"], q + "mlp.shared_expert.down_proj.weight": w[p + "shared_down"],
                    q + "mlp.shared_expert_gate.weight": w[p + "shared_expert_gate"]})
        for e in range(cfg.n_experts):
            out.update({q + f"mlp.experts.{e}.gate_proj.weight": w[p + "experts_in"][e, :F], q + f"mlp.experts.{e}.up_proj.weight": w[p + "experts_in"][e, F:],
                        q + f"mlp.experts.{e}.down_proj.weight": w[p + "experts_out"][e]})
    path.mkdir(parents=True, exist_ok=True)
    save_file({k: torch.from_numpy(np.ascontiguousarray(v, dtype=np.float32)) for k, v in out.items()}, str(path / "model.safetensors"),
              metadata={"format": "pt"})
    (path / "config.json").write_text(json.dumps(_header()))


def test_checkpoint_in_the_family_names_loads_and_generates(tmp_path):
    from poot_b200.driver.handle import ModelHandle
    from poot_b200.driver.sampler import SamplingParams
    from poot_b200.llm import LLM
    model = Registry.builtin().resolve_hf(_header())
    w = _weights(model, seed=6)
    _write_checkpoint(tmp_path / "ckpt", w, model.cfg)
    got = ModelHandle.load(str(tmp_path / "ckpt")).oracle_weights()
    assert sorted(got) == sorted(w)
    assert all(np.allclose(got[n], w[n], atol=1e-6) for n in w)            # norm scales come back through "- 1, + 1"
    prompt = [int(t) for t in np.random.default_rng(8).integers(0, 59, 21)]
    ref = Restated38(model.cfg, w)
    for t in prompt:
        logits = ref.token(t)
    want = []
    for _ in range(7):
        want.append(int(np.argmax(logits)))
        logits = ref.token(want[-1])
    llm = LLM.oracle(str(tmp_path / "ckpt"), rows=2, max_seq=48, num_blocks=16, prefill_chunk=16)
    assert llm.generate_tokens(prompt, SamplingParams(max_tokens=7, temperature=0.0, ignore_eos=True)) == want


def test_ngram_kernel_restatement_equals_the_hash_equation():
    """The host restatement the device test compares the n-gram kernel with, against the graph's ``ngram_hash``
    equation: pieces that start a sequence, continue one token at a time and carry the history between them."""
    import torch
    from poot_b200.ir.builder import Builder
    from poot_b200.oracle.eval import eval_graph
    from poot_b200.tensor import DType
    from poot_b200.utils import kernel_emulation as emu
    vocab, eos = 60, 59
    tb = ngram_tables(1, 3, 2, 50, 16, 7, vocab)
    toks = np.random.default_rng(0).integers(0, vocab, 11).astype(np.int32)
    toks[3] = eos
    b = Builder()
    win = b.slot("w", (2 + 11,), DType.I32, "token")
    b.output(b.ngram_hash(win, 2, tb.multipliers, tb.primes, tb.offsets, 2, eos), "ids")
    want = eval_graph(b.finish(), {"w": np.concatenate([[eos, eos], toks]).astype(np.int32)}).outputs["ids"]
    mult = torch.tensor([m - (1 << 64) if m >= 1 << 63 else m for m in tb.multipliers], dtype=torch.int64)
    primes, offsets = torch.tensor(tb.primes, dtype=torch.int32), torch.tensor(tb.offsets, dtype=torch.int32)
    hist, ids = torch.zeros(2, 2, dtype=torch.int32), torch.zeros(11, 4, dtype=torch.int32)
    for first, n in ((0, 4), (4, 1), (5, 1), (6, 5)):                 # a prompt chunk, two decode steps, another chunk
        emu.ngram_hash(torch.from_numpy(toks), hist, torch.tensor([[first, n, 1, first]], dtype=torch.int32), mult, primes, offsets, 2, eos,
                       vocab, ids)
    assert np.array_equal(ids.numpy(), want)
    assert hist[1].tolist() == [int(toks[-2]) ^ eos, int(toks[-1]) ^ eos] and hist[0].tolist() == [0, 0]


def test_sharded_fp8_ngram_table_loads_as_one_table(tmp_path):
    """The release stores an n-gram table as numbered E4M3 row-range shards under one scale: they load as one table at a
    byte per value whose decoded rows are ``code * scale``, and the model generates what it generates over those rows."""
    import torch
    from safetensors import safe_open
    from safetensors.torch import save_file
    from poot_b200.driver.handle import ModelHandle
    from poot_b200.load.hf_map import CheckpointLayout
    from poot_b200.quant.codec import e4m3_bits_to_f32
    model = Registry.builtin().resolve_hf(_header())
    w = _weights(model, seed=6)
    _write_checkpoint(tmp_path / "ckpt", w, model.cfg)
    path = str(tmp_path / "ckpt" / "model.safetensors")
    with safe_open(path, "pt") as f:
        tensors = {k: f.get_tensor(k) for k in f.keys()}
    scale = np.float32(0.03125)
    want = {}
    for k in [k for k in tensors if k.endswith("ngram_embedding.weight")]:
        t = tensors.pop(k)
        codes = (t / float(scale)).to(torch.float8_e4m3fn)
        cuts = [0, 1, t.shape[0] // 2, t.shape[0]]                     # a one-row shard, then two uneven ones
        for i, (lo, hi) in enumerate(zip(cuts[:-1], cuts[1:])):
            tensors[k.replace(".weight", f".shard_{i}.weight")] = codes[lo:hi].contiguous()
        tensors[k.replace(".weight", ".weight_scale")] = torch.tensor([float(scale)])
        layer = int(k.split("layers.")[1].split(".")[0])
        want[f"layers.{layer}.ple_table"] = e4m3_bits_to_f32(codes.view(torch.uint8).numpy()) * scale
    assert want
    save_file(tensors, path, metadata={"format": "pt"})
    h = ModelHandle.load(str(tmp_path / "ckpt"))
    for name, rows in want.items():
        pw = h.canonical[name]
        assert pw.format == "E4M3_CHANNEL" and pw.planar["weight"].dtype == np.uint8 and pw.planar["weight"].nbytes == rows.size
        assert np.array_equal(pw.to_f32(), rows)
    got = h.oracle_weights()
    assert all(np.array_equal(got[n], want[n]) for n in want)
    # a missing scale, or shards that do not count up from 0, are refused by name
    bad = {k: v for k, v in tensors.items() if not k.endswith("ngram_embedding.weight_scale")}
    save_file(bad, path, metadata={"format": "pt"})
    with pytest.raises(CheckpointLayout, match="weight_scale"):
        ModelHandle.load(str(tmp_path / "ckpt"))
    gap = {k: v for k, v in tensors.items() if ".shard_1." not in k}
    save_file(gap, path, metadata={"format": "pt"})
    with pytest.raises(CheckpointLayout, match="count up"):
        ModelHandle.load(str(tmp_path / "ckpt"))
