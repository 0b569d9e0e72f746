"""Makes tests/golden/sampling_probs.npz from the reference's own sampler.

Run once, on the CPU, with the reference's sources importable:

    PYTHONPATH=<reference checkout>/src python tests/golden/make_sampling_golden.py

``dli.sampling.sample`` draws with torch.multinomial, whose stream no other generator repeats; what can be
compared is the distribution it draws from.  The script stands in front of torch.multinomial, stores the
probabilities the reference hands it (put back into token order) for rows of random logits with different
temperatures, top-k and top-p, and stores the greedy choices of rows with ties.
tests/test_plain_vs_golden.py compares the plain sampler's ``filtered_probabilities`` with them.
"""

from pathlib import Path

import numpy as np
import torch

from dli.sampling import SamplingParams, make_generator, sample  # the reference

V = 97
SETTINGS = [(1.0, -1, 1.0), (0.7, -1, 1.0), (1.3, 5, 1.0), (0.9, -1, 0.8), (0.5, 12, 0.6), (2.0, 40, 0.95), (1.0, 1, 1.0), (0.8, 3, 0.1)]


def main():
    g = torch.Generator().manual_seed(11)
    logits = torch.randn(len(SETTINGS) * 3, V, generator=g) * 2.0
    logits[::3, 10:14] = logits[::3, 10:11]  # runs of equal values: the sort's order among them decides who is kept
    seen = []
    real = torch.multinomial

    def spy(probs, n, generator=None, **kw):
        seen.append(probs.clone())
        return real(probs, n, generator=generator, **kw)

    torch.multinomial = spy
    rows, probs, greedy = [], [], []
    try:
        for i in range(logits.shape[0]):
            t, k, p = SETTINGS[i % len(SETTINGS)]
            params = SamplingParams(temperature=t, top_k=k, top_p=p)
            seen.clear()
            token = sample(logits[i : i + 1], [params], [make_generator(5)])[0]
            if params.greedy:
                greedy.append((i, token))
                continue
            # the reference's probabilities are in sorted order: put them back into token order
            order = torch.sort(logits[i] / t, descending=True).indices
            row = torch.zeros(V)
            row[order] = seen[0]
            rows.append(i)
            probs.append(row.numpy())
    finally:
        torch.multinomial = real
    out = Path(__file__).resolve().parent / "sampling_probs.npz"
    np.savez(out, logits=logits.numpy(), settings=np.array(SETTINGS, dtype=np.float64), rows=np.array(rows), probs=np.stack(probs),
             greedy=np.array(greedy))
    print(len(rows), "stochastic rows,", len(greedy), "greedy rows ->", out, out.stat().st_size, "bytes")


if __name__ == "__main__":
    main()
