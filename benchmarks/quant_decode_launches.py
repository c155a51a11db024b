"""A few eager decode steps of the Q4_K / Q8_0 quantised Llama-3-8B stack (``layers`` layers), for a launch list.

    python benchmarks/quant_decode_launches.py [layers]
"""
import sys

import torch

sys.path.insert(0, ".")
from poot_b200.models.config import PRESETS  # noqa: E402
from poot_b200.runtime.engine import DecoderEngine  # noqa: E402
from poot_b200.runtime.session import FixedBatchSession  # noqa: E402
from poot_b200.runtime.weights import random_quant_weights  # noqa: E402

layers = int(sys.argv[1]) if len(sys.argv) > 1 else 4
cfg = PRESETS["llama-3-8b"]()
cfg.n_layers = layers
w = random_quant_weights(cfg, "cuda", seed=0)
max_len = 768
bps = max_len // 16
eng = DecoderEngine(w, num_blocks=bps, max_seqs=1, max_tokens=128, max_blocks_per_seq=bps, use_graphs=False)
s = FixedBatchSession(eng, 1, max_len)
s.len_t = torch.full((1,), 200, dtype=torch.int32)
for _ in range(4):
    s.decode([1])
torch.cuda.synchronize()
print("done")
