"""Vision-language family (Idefics3 / SmolVLM): tower + connector + text stack against the Hugging Face implementation,
image preprocessing against its processor, prompt expansion, and the ``caption`` command end to end."""
import json
import os

import numpy as np
import pytest

torch = pytest.importorskip("torch")
transformers = pytest.importorskip("transformers")
PIL = pytest.importorskip("PIL")

from poot_b200.models.image_prep import ImagePrep, image_prompt, preprocess, resize_for_encoder, resize_longest, split_geometry
from poot_b200.models.vision import VisionConfig, patchify, position_ids
from poot_b200.vlm import NotVisionModel, VisionLLM

SPECIALS = ["<|im_start|>", "<end_of_utterance>", "<fake_token_around_image>", "<global-img>", "<image>"] + \
           [f"<row_{r}_col_{c}>" for r in range(1, 4) for c in range(1, 4)]


def _tokenizer(path):
    """Byte-level tokenizer (256 byte tokens) with the front end's marker tokens added behind them."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    alphabet = pre_tokenizers.ByteLevel.alphabet()
    vocab = {ch: i for i, ch in enumerate(sorted(alphabet))}
    tk = Tokenizer(models.BPE(vocab=vocab, merges=[]))
    tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tk.decoder = decoders.ByteLevel()
    tk.add_special_tokens(SPECIALS)
    tk.save(os.path.join(path, "tokenizer.json"))
    with open(os.path.join(path, "tokenizer_config.json"), "w") as f:
        json.dump({"eos_token": "<end_of_utterance>"}, f)
    return tk


@pytest.fixture(scope="module")
def checkpoint(tmp_path_factory):
    from transformers import Idefics3Config, Idefics3ForConditionalGeneration
    d = str(tmp_path_factory.mktemp("idefics3"))
    tk = _tokenizer(d)
    image_token = tk.token_to_id("<image>")
    torch.manual_seed(0)
    cfg = Idefics3Config(
        text_config=dict(model_type="llama", hidden_size=128, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                         num_key_value_heads=2, vocab_size=tk.get_vocab_size(), max_position_embeddings=512, rms_norm_eps=1e-5),
        vision_config=dict(hidden_size=128, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, image_size=32,
                           patch_size=8, num_channels=3),
        scale_factor=2, image_token_id=image_token, pad_token_id=0)
    hf = Idefics3ForConditionalGeneration(cfg).eval()
    for p in hf.parameters():                                   # biases and norms away from their constant init
        if p.ndim == 1:
            p.data.add_(torch.randn_like(p) * 0.05)
    hf.save_pretrained(d, safe_serialization=True)
    with open(os.path.join(d, "preprocessor_config.json"), "w") as f:
        json.dump({"size": {"longest_edge": 64}, "max_image_size": {"longest_edge": 32}, "do_image_splitting": True,
                   "image_mean": [0.5] * 3, "image_std": [0.5] * 3, "rescale_factor": 1 / 255}, f)
    return d, hf, image_token


def test_logits_and_greedy_continuation_match_transformers(checkpoint):
    d, hf, image_token = checkpoint
    vlm = VisionLLM.load(d)
    rpi = vlm.vision.cfg.rows_per_image
    assert rpi == 4 and vlm.model.image_token == image_token
    rng = np.random.default_rng(0)
    pixels = rng.standard_normal((2, 3, 32, 32)).astype(np.float32)
    tokens = [5, 6] + [image_token] * rpi + [7] + [image_token] * rpi + [8, 9, 10]
    with torch.no_grad():
        out = hf(input_ids=torch.tensor([tokens]), pixel_values=torch.tensor(pixels)[None],
                 attention_mask=torch.ones(1, len(tokens), dtype=torch.long))
    want = out.logits[0, -1].numpy()
    sess = vlm._session(len(tokens))
    got = vlm.prefill(sess, tokens, pixels)[0]
    assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    # the image rows matter: the same tokens without them give different logits
    plain = vlm._session(len(tokens)).step(np.asarray([tokens], dtype=np.int32))[0]
    assert np.abs(plain - want).max() > 1e-3
    with torch.no_grad():
        gen = hf.generate(input_ids=torch.tensor([tokens]), pixel_values=torch.tensor(pixels)[None],
                          attention_mask=torch.ones(1, len(tokens), dtype=torch.long), max_new_tokens=6, do_sample=False,
                          eos_token_id=None, pad_token_id=0)
    assert vlm.generate(tokens, pixels, max_new=6) == gen[0, len(tokens):].tolist()


def test_image_rows_must_match_the_image_tokens(checkpoint):
    d, _, image_token = checkpoint
    vlm = VisionLLM.load(d)
    pixels = np.zeros((1, 3, 32, 32), dtype=np.float32)
    with pytest.raises(ValueError, match="image tokens"):
        vlm.prefill(vlm._session(16), [1, image_token, 2], pixels)
    with pytest.raises(ValueError, match="no image"):
        vlm.prefill(vlm._session(16), [1, image_token, 2], None)
    with pytest.raises(ValueError, match="tower takes"):
        vlm.encode_images(np.zeros((1, 3, 16, 16), dtype=np.float32))


def test_position_ids_and_patch_order():
    c = VisionConfig(image_size=32, patch=8)
    assert position_ids(c, 4, 4).tolist() == list(range(16))            # a full square image: the identity
    assert position_ids(c, 2, 2).tolist() == [0, 2, 8, 10]              # a smaller grid lands on every other bucket
    x = np.arange(2 * 3 * 16 * 16, dtype=np.float32).reshape(2, 3, 16, 16)
    p = patchify(x, 8)
    assert p.shape == (2, 4, 192)
    conv = torch.nn.functional.unfold(torch.tensor(x), kernel_size=8, stride=8).transpose(1, 2).numpy()
    assert np.array_equal(p, conv)
    ragged = np.arange(3 * 20 * 20, dtype=np.float32).reshape(1, 3, 20, 20)          # 20 / 8: the last 4 pixels are dropped
    conv = torch.nn.functional.unfold(torch.tensor(ragged), kernel_size=8, stride=8).transpose(1, 2).numpy()
    assert np.array_equal(patchify(ragged, 8), conv)


@pytest.mark.parametrize("hw", [(300, 500), (640, 200), (40, 40), (31, 77)])
def test_preprocessing_matches_the_reference_processor(hw):
    from PIL import Image
    from transformers.models.idefics3.image_processing_pil_idefics3 import Idefics3ImageProcessorPil
    from transformers.models.idefics3.processing_idefics3 import get_image_prompt_string
    rng = np.random.default_rng(1)
    img = Image.fromarray(rng.integers(0, 255, (*hw, 3), dtype=np.uint8))
    for tile, longest in ((64, 256), (32, 50)):
        ip = Idefics3ImageProcessorPil(size={"longest_edge": longest}, max_image_size={"longest_edge": tile},
                                       image_mean=[0.5] * 3, image_std=[0.5] * 3)
        out = ip(images=[img], return_tensors="np", return_row_col_info=True)
        prep = ImagePrep(longest_edge=longest, tile=tile)
        fr = preprocess(img, prep)
        assert (fr.rows, fr.cols) == (out["rows"][0][0], out["cols"][0][0])
        assert fr.pixels.shape == out["pixel_values"][0].shape
        assert np.abs(fr.pixels - out["pixel_values"][0]).max() < 1e-6
        want = get_image_prompt_string(fr.rows, fr.cols, 4, "<fake_token_around_image>", "<image>", "<global-img>")
        assert image_prompt(prep, fr.rows, fr.cols, 4) == want


def test_resize_geometry():
    assert resize_longest(300, 500, 100) == (60, 100)
    assert resize_longest(501, 100, 100) == (100, 20)               # odd short edge rounds up to even
    assert resize_for_encoder(60, 100, 32) == (96, 128)
    assert split_geometry(96, 128, 32) == (3, 4) and split_geometry(32, 32, 32) == (0, 0)
    one = preprocess(__import__("PIL.Image", fromlist=["x"]).new("RGB", (20, 20)), ImagePrep(longest_edge=32, tile=32))
    assert one.pixels.shape == (1, 3, 32, 32) and (one.rows, one.cols) == (0, 0)
    unsplit = preprocess(__import__("PIL.Image", fromlist=["x"]).new("L", (90, 50)), ImagePrep(longest_edge=64, tile=32, split=False))
    assert unsplit.pixels.shape == (1, 3, 32, 32)


def test_caption_command_end_to_end(checkpoint, tmp_path, capsys):
    from PIL import Image
    from poot_b200.cli.__main__ import main
    d, hf, image_token = checkpoint
    rng = np.random.default_rng(2)
    path = str(tmp_path / "picture.png")
    img = Image.fromarray(rng.integers(0, 255, (40, 60, 3), dtype=np.uint8))
    img.save(path)
    vlm = VisionLLM.load(d)
    tokens, pixels = vlm.prepare("What is this?", img)
    # 60x40 scales to 64x44 -> rounds up to 64x64 -> 2x2 tiles plus the global frame
    assert pixels.shape == (5, 3, 32, 32) and tokens.count(image_token) == 5 * vlm.vision.cfg.rows_per_image
    text = vlm.tokenizer.tk.decode(tokens, skip_special_tokens=False)
    assert text.startswith("<|im_start|>User:<fake_token_around_image><row_1_col_1><image>") and text.endswith("Assistant:")
    assert "<global-img>" in text and "What is this?<end_of_utterance>" in text
    with torch.no_grad():
        gen = hf.generate(input_ids=torch.tensor([tokens]), pixel_values=torch.tensor(pixels)[None],
                          attention_mask=torch.ones(1, len(tokens), dtype=torch.long), max_new_tokens=5, do_sample=False,
                          eos_token_id=None, pad_token_id=0)
    want = gen[0, len(tokens):].tolist()
    assert vlm.generate(tokens, pixels, max_new=5) == want
    assert main(["caption", d, path, "What is this?", "-n", "5"]) == 0
    out = capsys.readouterr().out
    eos = vlm.tokenizer.eos
    shown = want[:want.index(eos)] if eos in want else want
    from poot_b200.text.codec import StreamDecoder
    dec = StreamDecoder(vlm.tokenizer)
    streamed = "".join(dec.push(t) for t in shown) + dec.flush()
    assert out == streamed + "\n"
    assert main(["caption", d, str(tmp_path / "missing.png")]) == 1
    assert main(["caption", d]) == 2


def _hf_greedy(hf, tokens, pixels, n):
    with torch.no_grad():
        gen = hf.generate(input_ids=torch.tensor([tokens]), pixel_values=torch.tensor(pixels)[None],
                          attention_mask=torch.ones(1, len(tokens), dtype=torch.long), max_new_tokens=n, do_sample=False,
                          eos_token_id=None, pad_token_id=0)
    return gen[0, len(tokens):].tolist()


def test_image_rows_through_the_driver_chunked_prefill_and_prefix_cache(checkpoint):
    """Image rows ride the ordinary driver: prefill in pieces of 16 tokens cuts the image runs across steps, and the
    prefix cache tells two images behind identical placeholder tokens apart."""
    d, hf, image_token = checkpoint
    vlm = VisionLLM.load(d, backend="oracle", rows=2, max_seq=128, prefill_chunk=16, num_blocks=32)
    rpi = vlm.vision.cfg.rows_per_image
    rng = np.random.default_rng(3)
    a = rng.standard_normal((5, 3, 32, 32)).astype(np.float32)
    b = rng.standard_normal((5, 3, 32, 32)).astype(np.float32)
    tokens = [5, 6, 7] + [image_token] * (3 * rpi) + [9] + [image_token] * (2 * rpi) + list(range(20, 33))
    assert len(tokens) > 32                                         # at least two full blocks can be shared
    want_a, want_b = _hf_greedy(hf, tokens, a, 5), _hf_greedy(hf, tokens, b, 5)
    assert want_a != want_b
    drv = vlm.llm.driver
    assert vlm.generate(tokens, a, max_new=5) == want_a
    hits = drv.stats["prefix_hit_tokens"]
    assert vlm.generate(tokens, b, max_new=5) == want_b             # same tokens, other image: no shared prefix
    assert drv.stats["prefix_hit_tokens"] == hits
    assert vlm.generate(tokens, a, max_new=5) == want_a             # the first image again: its blocks are reused
    assert drv.stats["prefix_hit_tokens"] >= hits + 32
    from poot_b200.driver.driver import DriverError
    with pytest.raises(DriverError, match="ascending"):
        drv.open(tokens, embeds=(np.array([4, 3]), np.zeros((2, 128), np.float32)))


def test_image_rows_on_the_emulated_device_engine(checkpoint):
    """The device engine's program (kernels restated on the host, bf16): the staged rows replace the image tokens'
    embeddings after the gather, in chunked prefill too."""
    from poot_b200.utils.kernel_emulation import emulated_kernels
    d, hf, image_token = checkpoint
    rpi = 4
    rng = np.random.default_rng(4)
    pixels = rng.standard_normal((3, 3, 32, 32)).astype(np.float32)
    tokens = [5, 6] + [image_token] * (3 * rpi) + [8, 9, 10, 11, 12, 13, 14]
    want = _hf_greedy(hf, tokens, pixels, 6)
    with emulated_kernels():
        vlm = VisionLLM.load(d, backend="device", device="cpu", rows=1, max_seq=64, prefill_chunk=16, num_blocks=8)
        assert vlm.vision_engine is not None                      # 32-wide heads: the tower runs on the engine too
        got = vlm.generate(tokens, pixels, max_new=6)
        assert vlm.vision_engine.launches == 4 + 13 * 2 + 3
        eng = vlm.llm.engine
        assert any(k[-2] for k in eng.launches_per_step), "no step ran with rows in place of embeddings"
        blind = vlm.llm.generate_tokens(tokens, __import__("poot_b200").SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    agree = 0
    for x, y in zip(got, want):
        if x != y:
            break
        agree += 1
    assert agree >= 2, (got, want)
    assert blind != got                                               # without the rows the continuation is another one


def test_chat_completions_take_image_url_parts(checkpoint):
    """An OpenAI-style chat request with a base64 ``image_url`` part: the server expands the placeholder, runs the tower
    and opens the sequence with the image rows; the completion is the one ``transformers`` generates for that prompt."""
    import base64
    import http.client
    import io
    from PIL import Image
    from poot_b200.llm import LLM
    from poot_b200.serve import Metrics, ServeConfig, ServeEngine, Server, ServerState
    d, hf, image_token = checkpoint
    llm = LLM.oracle(d, rows=2, max_seq=256, num_blocks=40, prefill_chunk=32)
    cfg = ServeConfig(model=d, addr="127.0.0.1:0", rows=2)
    eng = ServeEngine(llm.driver, llm.tokenizer, Metrics(), 8, cfg.max_queue_wait_secs)
    state = ServerState(eng, cfg, "tiny-vlm", family="idefics3")
    state.vision = VisionLLM(llm.handle, llm.tokenizer, None, llm)
    srv = Server(state)
    eng.start()
    srv.start()

    def post(body):
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=60)
        c.request("POST", "/v1/chat/completions", json.dumps(body).encode(), {"Content-Type": "application/json"})
        r = c.getresponse()
        out = r.status, json.loads(r.read())
        c.close()
        return out
    try:
        img = Image.fromarray(np.random.default_rng(6).integers(0, 255, (30, 30, 3), dtype=np.uint8))
        buf = io.BytesIO()
        img.save(buf, format="PNG")
        url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
        msgs = [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}}, {"type": "text", "text": "What?"}]}]
        tokens, pixels = state.vision.prepare_messages(msgs)
        want = _hf_greedy(hf, tokens, pixels, 4)
        st, body = post({"messages": msgs, "max_tokens": 4, "temperature": 0, "ignore_eos": True})
        assert st == 200, body
        assert body["usage"]["prompt_tokens"] == len(tokens) and body["usage"]["completion_tokens"] == 4
        from poot_b200.text.codec import StreamDecoder
        eos = llm.driver.eos_token
        assert body["choices"][0]["message"]["content"] == llm.tokenizer.decode([t for t in want if t != eos])
        st, body = post({"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "https://example.com/a.png"}}]}]})
        assert st == 400 and "data: URL" in body["error"]["message"]
        st, body = post({"messages": [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": "data:image/png;base64,AAAA"}}]}]})
        assert st == 400 and "decode" in body["error"]["message"]
        state.vision = None
        st, body = post({"messages": msgs, "max_tokens": 2})
        assert st == 400 and "no vision front end" in body["error"]["message"]
    finally:
        srv.shutdown()


def test_text_checkpoints_have_no_front_end(tmp_path):
    from transformers import LlamaConfig, LlamaForCausalLM
    d = str(tmp_path / "llama")
    LlamaForCausalLM(LlamaConfig(hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=2,
                                 num_key_value_heads=2, vocab_size=64)).save_pretrained(d, safe_serialization=True)
    with pytest.raises(NotVisionModel):
        VisionLLM.load(d)


# ---- Qwen2.5-VL ----------------------------------------------------------------------------------------------------
QWEN_SPECIALS = ["<|im_start|>", "<|im_end|>", "<|vision_start|>", "<|vision_end|>", "<|image_pad|>", "<|video_pad|>"]


@pytest.fixture(scope="module")
def qwen_checkpoint(tmp_path_factory):
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    d = str(tmp_path_factory.mktemp("qwen_vl"))
    vocab = {ch: i for i, ch in enumerate(sorted(pre_tokenizers.ByteLevel.alphabet()))}
    tk = Tokenizer(models.BPE(vocab=vocab, merges=[]))
    tk.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tk.decoder = decoders.ByteLevel()
    tk.add_special_tokens(QWEN_SPECIALS)
    tk.save(os.path.join(d, "tokenizer.json"))
    with open(os.path.join(d, "tokenizer_config.json"), "w") as f:
        json.dump({"eos_token": "<|im_end|>"}, f)
    ids = {t: tk.token_to_id(t) for t in QWEN_SPECIALS}
    torch.manual_seed(0)
    cfg = Qwen2_5_VLConfig(
        text_config=dict(hidden_size=64, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         vocab_size=tk.get_vocab_size(), max_position_embeddings=512,
                         rope_parameters={"rope_type": "default", "mrope_section": [2, 3, 3], "rope_theta": 10000.0}),
        # one position token per second: this transformers version multiplies an image's start position by the rate
        vision_config=dict(depth=3, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, window_size=16, fullatt_block_indexes=[1],
                           out_hidden_size=64, tokens_per_second=1),
        image_token_id=ids["<|image_pad|>"], video_token_id=ids["<|video_pad|>"], vision_start_token_id=ids["<|vision_start|>"],
        vision_end_token_id=ids["<|vision_end|>"])
    hf = Qwen2_5_VLForConditionalGeneration(cfg).eval()
    for p in hf.parameters():
        if p.ndim == 1:
            p.data.add_(torch.randn_like(p) * 0.1)
    hf.save_pretrained(d, safe_serialization=True)
    with open(os.path.join(d, "preprocessor_config.json"), "w") as f:
        json.dump({"size": {"shortest_edge": 16 * 16, "longest_edge": 8 * 8 * 40}, "patch_size": 4, "merge_size": 2,
                   "temporal_patch_size": 2}, f)
    with open(os.path.join(d, "video_preprocessor_config.json"), "w") as f:
        json.dump({"size": {"shortest_edge": 8 * 8, "longest_edge": 8 * 8 * 12}, "fps": 2.0, "min_frames": 4, "max_frames": 16}, f)
    return d, hf, ids


def _qwen_greedy(hf, tokens, images, image_token, n):
    ids = torch.tensor([tokens])
    with torch.no_grad():
        gen = hf.generate(input_ids=ids, pixel_values=torch.tensor(images.patches), image_grid_thw=torch.tensor(images.grids),
                          attention_mask=torch.ones_like(ids), mm_token_type_ids=(ids == image_token).long(), max_new_tokens=n,
                          do_sample=False, eos_token_id=None, pad_token_id=0)
    return gen[0, len(tokens):].tolist()


def test_qwen_vl_tower_logits_and_generation_match_transformers(qwen_checkpoint):
    from poot_b200.models.image_prep import QwenImages
    d, hf, ids = qwen_checkpoint
    vlm = VisionLLM.load(d)
    IMG = ids["<|image_pad|>"]
    assert vlm.qwen and vlm.model.image_token == IMG and vlm.handle.cfg.mrope_sections == [2, 3, 3]
    grids = [(1, 8, 12), (1, 4, 6)]                  # two images: 6 windows of 2x2 merged cells, and 2x... a ragged edge
    n = sum(t * h * w for t, h, w in grids)
    images = QwenImages(np.random.default_rng(0).standard_normal((n, vlm.vision.cfg.patch_dim)).astype(np.float32), grids)
    with torch.no_grad():
        want_rows = hf.model.visual(torch.tensor(images.patches), grid_thw=torch.tensor(grids)).pooler_output.numpy()
    rows = vlm.encode_images(images)
    assert rows.shape == (24 + 6, 64) and np.abs(rows - want_rows).max() < 1e-5
    tokens = [5, 6, ids["<|vision_start|>"]] + [IMG] * 24 + [ids["<|vision_end|>"], 7, ids["<|vision_start|>"]] + [IMG] * 6 + \
             [ids["<|vision_end|>"], 8, 9, 10, 11]
    t = torch.tensor([tokens])
    with torch.no_grad():
        out = hf(input_ids=t, pixel_values=torch.tensor(images.patches), image_grid_thw=torch.tensor(grids),
                 attention_mask=torch.ones_like(t), mm_token_type_ids=(t == IMG).long())
    want = out.logits[0, -1].numpy()
    got = vlm.prefill(vlm._session(len(tokens)), tokens, images)[0]
    assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    assert vlm.rope_delta == (2 + 1 + 6 + 2 + 1 + 3 + 5) - len(tokens)          # an image advances by its longer merged edge
    assert vlm.generate(tokens, images, max_new=6) == _qwen_greedy(hf, tokens, images, IMG, 6)
    # without images the three streams are equal and the stack is the plain Qwen2 one
    plain = [5, 6, 7, 8, 9, 10]
    with torch.no_grad():
        want = hf(input_ids=torch.tensor([plain])).logits[0, -1].numpy()
    assert np.abs(vlm.prefill(vlm._session(16), plain, None)[0] - want).max() < 1e-5
    # through the serving driver: chunked prefill cuts the image runs, decode continues at index + delta
    served = VisionLLM.load(d, backend="oracle", rows=2, max_seq=128, prefill_chunk=16, num_blocks=32)
    assert served.llm is not None and served.generate(tokens, images, max_new=6) == _qwen_greedy(hf, tokens, images, IMG, 6)
    assert served.generate(plain, None, max_new=4) == vlm.generate(plain, None, max_new=4)


def test_qwen_vl_chat_completions_with_an_image(qwen_checkpoint):
    """The served path of the sectioned-rope family: an ``image_url`` part becomes image rows and three rotary position
    streams on the scheduler's job; the completion is the one ``transformers`` generates."""
    import base64
    import http.client
    import io
    from PIL import Image
    from poot_b200.llm import LLM
    from poot_b200.serve import Metrics, ServeConfig, ServeEngine, Server, ServerState
    d, hf, ids = qwen_checkpoint
    llm = LLM.oracle(d, rows=2, max_seq=256, num_blocks=40, prefill_chunk=32)
    cfg = ServeConfig(model=d, addr="127.0.0.1:0", rows=2)
    eng = ServeEngine(llm.driver, llm.tokenizer, Metrics(), 8, cfg.max_queue_wait_secs)
    state = ServerState(eng, cfg, "tiny-qwen-vl", family="qwen_vl")
    state.vision = VisionLLM(llm.handle, llm.tokenizer, None, llm)
    srv = Server(state)
    eng.start()
    srv.start()
    try:
        img = Image.fromarray(np.random.default_rng(8).integers(0, 255, (24, 40, 3), dtype=np.uint8))
        buf = io.BytesIO()
        img.save(buf, format="PNG")
        url = "data:image/png;base64," + base64.b64encode(buf.getvalue()).decode()
        msgs = [{"role": "user", "content": [{"type": "image_url", "image_url": {"url": url}}, {"type": "text", "text": "What?"}]}]
        tokens, images = state.vision.prepare_messages(msgs)
        want = _qwen_greedy(hf, tokens, images, ids["<|image_pad|>"], 4)
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=60)
        c.request("POST", "/v1/chat/completions", json.dumps({"messages": msgs, "max_tokens": 4, "temperature": 0, "ignore_eos": True}).encode(),
                  {"Content-Type": "application/json"})
        r = c.getresponse()
        body = json.loads(r.read())
        c.close()
        assert r.status == 200, body
        assert body["usage"]["prompt_tokens"] == len(tokens)
        eos = llm.driver.eos_token
        assert body["choices"][0]["message"]["content"] == llm.tokenizer.decode([t for t in want if t != eos])
    finally:
        srv.shutdown()


def test_mrope_positions():
    from poot_b200.models.vision import mrope_positions
    I = 99
    pos = mrope_positions([1, 2] + [I] * 6 + [3, 4], I, [(1, 4, 6)], 2)          # 2 x 3 merged cells starting at 2
    assert pos[0].tolist() == [0, 1, 2, 2, 2, 2, 2, 2, 5, 6]
    assert pos[1].tolist() == [0, 1, 2, 2, 2, 3, 3, 3, 5, 6]
    assert pos[2].tolist() == [0, 1, 2, 3, 4, 2, 3, 4, 5, 6]
    assert mrope_positions([4, 5, 6], I, [], 2).tolist() == [[0, 1, 2]] * 3
    with pytest.raises(ValueError, match="fewer than"):
        mrope_positions([1] + [I] * 5, I, [(1, 4, 6)], 2)
    with pytest.raises(ValueError, match="more image runs"):
        mrope_positions([I] * 6 + [1] + [I] * 6, I, [(1, 4, 6)], 2)
    with pytest.raises(ValueError, match="2 images for 1"):
        mrope_positions([I] * 6, I, [(1, 4, 6), (1, 4, 6)], 2)


@pytest.mark.parametrize("hw", [(300, 500), (64, 40), (1000, 900), (30, 31)])
def test_qwen_preprocessing_matches_the_reference_processor(hw):
    from PIL import Image
    from transformers.models.qwen2_vl.image_processing_pil_qwen2_vl import Qwen2VLImageProcessorPil
    from poot_b200.models.image_prep import QwenImagePrep, qwen_preprocess, smart_resize
    img = Image.fromarray(np.random.default_rng(0).integers(0, 255, (*hw, 3), dtype=np.uint8))
    for patch, lo, hi in ((14, 56 * 56, 28 * 28 * 1280), (4, 16 * 16, 8 * 8 * 40)):
        ip = Qwen2VLImageProcessorPil(patch_size=patch, merge_size=2, temporal_patch_size=2, size={"shortest_edge": lo, "longest_edge": hi})
        out = ip(images=[img], return_tensors="np")
        got = qwen_preprocess(img, QwenImagePrep(patch=patch, min_pixels=lo, max_pixels=hi))
        assert got.grids == [tuple(int(x) for x in out["image_grid_thw"][0])]
        assert got.patches.shape == out["pixel_values"].shape and np.abs(got.patches - out["pixel_values"]).max() < 2e-6
    assert smart_resize(30, 31, 28, 56 * 56, 10 ** 6) == (56, 84) and smart_resize(1000, 900, 8, 256, 2560) == (48, 48)
    with pytest.raises(ValueError, match="aspect"):
        smart_resize(10, 2001, 28, 1, 10 ** 9)


def test_qwen_caption_command(qwen_checkpoint, tmp_path, capsys):
    from PIL import Image
    from poot_b200.cli.__main__ import main
    from poot_b200.text.codec import StreamDecoder
    d, hf, ids = qwen_checkpoint
    path = str(tmp_path / "picture.png")
    img = Image.fromarray(np.random.default_rng(3).integers(0, 255, (40, 60, 3), dtype=np.uint8))
    img.save(path)
    vlm = VisionLLM.load(d)
    tokens, images = vlm.prepare("What is this?", img)
    assert images.grids == [(1, 10, 16)] and tokens.count(ids["<|image_pad|>"]) == 40
    text = vlm.tokenizer.tk.decode(tokens, skip_special_tokens=False)
    assert "<|im_start|>user\n<|vision_start|><|image_pad|>" in text and text.endswith("What is this?<|im_end|>\n<|im_start|>assistant\n")
    want = _qwen_greedy(hf, tokens, images, ids["<|image_pad|>"], 5)
    assert vlm.generate(tokens, images, max_new=5) == want
    assert main(["caption", d, path, "What is this?", "-n", "5", "--backend", "oracle"]) == 0
    out = capsys.readouterr().out
    eos = vlm.tokenizer.eos
    shown = want[:want.index(eos)] if eos in want else want
    dec = StreamDecoder(vlm.tokenizer)
    assert out == "".join(dec.push(t) for t in shown) + dec.flush() + "\n"


def test_qwen_vl_images_on_the_emulated_device_engine(tmp_path):
    """The device engine's program under a sectioned rope: the per-token rotary rows staged by ``bind_rope_streams``
    (time / row / column streams by channel section) and the image rows staged by ``bind_embeds``, in chunked prefill
    and decode, against ``transformers`` greedy generation (bf16 on the engine side: the first tokens must agree)."""
    from transformers import Qwen2_5_VLConfig, Qwen2_5_VLForConditionalGeneration
    from poot_b200.models.image_prep import QwenImages
    from poot_b200.utils.kernel_emulation import emulated_kernels
    torch.manual_seed(0)
    cfg = Qwen2_5_VLConfig(
        text_config=dict(hidden_size=128, intermediate_size=96, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                         vocab_size=300, max_position_embeddings=256,
                         rope_parameters={"rope_type": "default", "mrope_section": [4, 6, 6], "rope_theta": 10000.0}),
        vision_config=dict(depth=2, hidden_size=32, intermediate_size=48, num_heads=2, in_channels=3, patch_size=4,
                           spatial_merge_size=2, temporal_patch_size=2, window_size=16, fullatt_block_indexes=[1],
                           out_hidden_size=128, tokens_per_second=1),
        image_token_id=290, video_token_id=291, vision_start_token_id=292, vision_end_token_id=293)
    hf = Qwen2_5_VLForConditionalGeneration(cfg).eval()
    with torch.no_grad():
        for p in hf.parameters():
            if p.ndim == 1:
                p.add_(torch.randn_like(p) * 0.1)
    d = str(tmp_path)
    hf.save_pretrained(d, safe_serialization=True)
    grids = [(1, 8, 12)]
    images = QwenImages(np.random.default_rng(5).standard_normal((96, 96)).astype(np.float32), grids)
    tokens = [5, 6, 292] + [290] * 24 + [293, 8, 9, 10, 11, 12]
    want = _qwen_greedy(hf, tokens, images, 290, 6)
    with emulated_kernels():
        vlm = VisionLLM.load(d, backend="device", device="cpu", rows=1, max_seq=64, prefill_chunk=16, num_blocks=8)
        got = vlm.generate(tokens, images, max_new=6)
        keys = list(vlm.llm.engine.launches_per_step)
        assert any(k[-1] and k[-2] for k in keys) and any(k[-1] and not k[-2] for k in keys)   # image chunks, then plain ones
        eng = vlm.llm.engine
        streams = torch.tensor([[3, 3, 3, 9], [3, 4, 5, 9], [7, 3, 2, 9]], dtype=torch.int32)
        eng.bind_rope_streams(streams)
        owner = [0] * 4 + [1] * 6 + [2] * 6                                  # sections [4, 6, 6] of the 16 channel pairs
        for t in range(4):
            for j in (0, 3, 4, 9, 10, 15):
                assert eng.rope_cos_tok[t, j] == eng.cos[int(streams[owner[j], t]), j]
                assert eng.rope_sin_tok[t, j] == eng.sin[int(streams[owner[j], t]), j]
    agree = 0
    for x, y in zip(got, want):
        if x != y:
            break
        agree += 1
    assert agree >= 2, (got, want)


def _apng(frames, ms):
    import io
    buf = io.BytesIO()
    frames[0].save(buf, format="PNG", save_all=True, append_images=frames[1:], duration=ms, loop=0)
    return buf.getvalue()


def test_video_frame_sampling_and_time_positions():
    """Uniform sampling at two frames per second of source, clamped and cut to whole temporal steps; a video's time
    stream advances by ``floor(step * seconds per step * positions per second)`` and the text continues past it."""
    from poot_b200.models.image_prep import QwenVideoPrep, sample_video_frames
    from poot_b200.models.vision import mrope_positions
    p = QwenVideoPrep()
    assert sample_video_frames(30, 10.0, p) == [0, 5, 10, 15, 20, 25]            # 3 s at 2 per second
    assert sample_video_frames(100, 50.0, p) == [0, 25, 50, 75]                  # 2 s would be 4 frames: the minimum
    assert sample_video_frames(3, 1.0, p) == [0, 1]                               # never more than the clip, whole steps only
    assert sample_video_frames(1, 1.0, p) == [0]
    assert len(sample_video_frames(16 * 1024, 1.0, QwenVideoPrep(max_frames=768))) == 768
    for bad in (0.0, float("nan"), float("inf"), -1.0):
        with pytest.raises(ValueError):
            sample_video_frames(10, bad, p)
    with pytest.raises(ValueError):
        sample_video_frames(0, 1.0, p)
    V, I = 98, 99
    # three temporal steps of 2 x 2 merged cells, two seconds per step, 25 positions per second: 0, 50, 100
    pos = mrope_positions([7] + [V] * 12 + [8, 9], I, [(3, 4, 4)], 2, video_token=V, seconds_per_step=[2.0], tokens_per_second=25)
    assert pos[0].tolist() == [0] + [1] * 4 + [51] * 4 + [101] * 4 + [102, 103]
    assert pos[1].tolist() == [0] + [1, 1, 2, 2] * 3 + [102, 103]
    assert pos[2].tolist() == [0] + [1, 2, 1, 2] * 3 + [102, 103]
    # an image and a video in one prompt, each at its own kind of run
    both = mrope_positions([I] * 4 + [5] + [V] * 8, I, [(1, 4, 4), (2, 4, 4)], 2, video_token=V, seconds_per_step=[None, 0.5], tokens_per_second=2)
    assert both[0].tolist() == [0] * 4 + [2] + [3] * 4 + [4] * 4
    with pytest.raises(ValueError, match="is a video"):
        mrope_positions([I] * 8, I, [(2, 4, 4)], 2, video_token=V, seconds_per_step=[1.0])
    with pytest.raises(ValueError, match="without a video"):
        mrope_positions([V] * 4, I, [(1, 4, 4)], 2, video_token=V, seconds_per_step=[None])


def test_qwen_vl_video_rows_and_logits(qwen_checkpoint):
    """A clip through the front end: an animated PNG is sampled, patched two frames per temporal step and written as
    video placeholders; the tower's rows equal ``transformers``' video features, and with the same position streams the
    logits equal its forward."""
    from PIL import Image
    from poot_b200.models.image_prep import read_apng
    d, hf, ids = qwen_checkpoint
    vlm = VisionLLM.load(d)
    VID = ids["<|video_pad|>"]
    assert vlm.vision.cfg.video_token == VID and vlm.vision.cfg.tokens_per_second == 1.0
    rng = np.random.default_rng(0)
    frames = [Image.fromarray(rng.integers(0, 255, (24, 32, 3), dtype=np.uint8)) for _ in range(10)]
    data = _apng(frames, 250)                                                 # 4 frames per second: 2.5 s, five kept
    clip = read_apng(data)
    assert len(clip.frames) == 10 and abs(clip.fps - 4.0) < 1e-9 and clip.timestamps[:3] == [0.0, 0.25, 0.5]
    import base64
    url = "data:image/apng;base64," + base64.b64encode(data).decode()
    tokens, pixels = vlm.prepare_messages([{"role": "user", "content": [{"type": "video_url", "video_url": {"url": url}},
                                                                        {"type": "text", "text": "what moves?"}]}])
    (t, h, w), = pixels.grids
    assert t == 2 and pixels.seconds is not None and abs(pixels.seconds[0] - 2 / (4 / 2.5)) < 1e-9      # 4 kept frames over 2.5 s
    n = t * h * w // 4
    assert tokens.count(VID) == n and tokens.count(ids["<|image_pad|>"]) == 0
    with torch.no_grad():
        want_rows = hf.model.visual(torch.tensor(pixels.patches), grid_thw=torch.tensor(pixels.grids)).pooler_output.numpy()
    rows = vlm.encode_images(pixels)
    assert rows.shape == (n, 64) and np.abs(rows - want_rows).max() < 1e-5
    rope = vlm.rope_inputs(tokens, pixels)
    first = tokens.index(VID)
    step = int(np.floor(pixels.seconds[0] * 1.0))
    assert rope[0, first] == first and rope[0, first + n - 1] == first + step                       # the second temporal step is later in time
    ids_t = torch.tensor([tokens])
    with torch.no_grad():
        out = hf(input_ids=ids_t, pixel_values_videos=torch.tensor(pixels.patches), video_grid_thw=torch.tensor(pixels.grids),
                 attention_mask=torch.ones_like(ids_t), position_ids=torch.tensor(rope)[:, None, :].long())
    want = out.logits[0, -1].numpy()
    got = vlm.prefill(vlm._session(len(tokens)), tokens, pixels)[0]
    assert np.abs(got - want).max() <= 2e-5 * max(1.0, np.abs(want).max())
    # through the serving driver: the video rows ride the same embedding path as image rows
    served = VisionLLM.load(d, backend="oracle", rows=2, max_seq=256, prefill_chunk=16, num_blocks=48)
    assert served.generate(tokens, pixels, max_new=4) == vlm.generate(tokens, pixels, max_new=4)
    with pytest.raises(ValueError, match="data: URL"):
        vlm.prepare_messages([{"role": "user", "content": [{"type": "video_url", "video_url": {"url": "https://example.com/a.png"}}]}])


def test_qwen_caption_command_takes_an_animated_png(qwen_checkpoint, tmp_path, capsys):
    from PIL import Image
    from poot_b200.cli.caption import main_caption
    d, hf, ids = qwen_checkpoint
    rng = np.random.default_rng(1)
    frames = [Image.fromarray(rng.integers(0, 255, (16, 24, 3), dtype=np.uint8)) for _ in range(8)]
    path = str(tmp_path / "clip.png")
    with open(path, "wb") as f:
        f.write(_apng(frames, 500))
    assert main_caption([d, path, "what moves?", "-n", "4", "--backend", "oracle"]) == 0
    out = capsys.readouterr().out.rstrip("\n")
    vlm = VisionLLM.load(d)
    from poot_b200.models.image_prep import read_apng
    tokens, pixels = vlm.prepare("what moves?", read_apng(open(path, "rb").read()))
    assert pixels.grids[0][0] == 4 and tokens.count(ids["<|video_pad|>"]) > 0          # 4 s at two frames per second, two per step
    want = vlm.generate(tokens, pixels, max_new=4, eos=[vlm.handle.cfg.eos_token])
    assert out == vlm.tokenizer.decode(want)
