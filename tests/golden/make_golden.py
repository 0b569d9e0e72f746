"""Makes the golden arrays under tests/golden/ from the reference's own model code.

Run once, on the CPU, with the reference's sources importable:

    PYTHONPATH=<reference checkout>/src python tests/golden/make_golden.py

For each tiny configuration it writes a random-weights model folder into a
temporary directory (this repository's writer, seeds as in tests/tiny_configs.py),
loads it with the reference's ``dli.model.load_model`` in float32, and stores

  <name>.npz: token ids, logits of the whole sequence at a few positions,
              the reference's inverse frequencies, 16 greedy tokens, and a
              checksum of the weights (so a changed random stream is noticed).

tests/test_plain_vs_golden.py compares the plain implementation with these.
"""

import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import dli_b200  # noqa: E402
from dli.generate import greedy_generate  # noqa: E402  (the reference)
from dli.model import load_model  # noqa: E402  (the reference)
from tests.tiny_configs import TINY  # noqa: E402

POSITIONS = {"tiny_a": [0, 1, 4, 16, 32], "tiny_b": [0, 1, 7, 31, 63, 64, 89], "tiny_c": [0, 3, 20, 47]}


def main() -> None:
    out_dir = Path(__file__).resolve().parent
    for name, (cfg, seed, _page) in TINY.items():
        with tempfile.TemporaryDirectory() as tmp:
            dli_b200.write_model_dir(tmp, cfg, seed)
            model = load_model(tmp, dtype=torch.float32, device="cpu")
        n = POSITIONS[name][-1] + 1
        g = torch.Generator().manual_seed(100 + seed)
        ids = torch.randint(0, cfg["vocab_size"], (n,), generator=g)
        with torch.inference_mode():
            logits = model(ids, torch.arange(n))
        greedy = greedy_generate(model, ids[:9].tolist(), 16)
        checksum = sum(float(p.double().abs().sum()) for p in model.state_dict().values())
        np.savez(
            out_dir / f"{name}.npz",
            token_ids=ids.numpy().astype(np.int32),
            positions=np.array(POSITIONS[name], dtype=np.int32),
            logits=logits[POSITIONS[name]].numpy().astype(np.float32),
            inv_freq=model.inv_freq.numpy().astype(np.float32),
            greedy=np.array(greedy, dtype=np.int32),
            weight_checksum=np.array(checksum, dtype=np.float64),
        )
        print(name, "logits", tuple(logits.shape), "max", float(logits.abs().max()), "greedy", greedy[:6])


if __name__ == "__main__":
    main()
