"""Generates tests/golden/sampling_cases.json: token ids drawn by the reference's own sampler
(scripts/demo_support/api.py:_sample_next_token) from seeded logits under a seeded generator.  Needs a
FlashSVD checkout; run once in the build container:

    python tests/golden/make_sampling_golden.py --reference <FlashSVD checkout>
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch

OUT = Path(__file__).resolve().parent / "sampling_cases.json"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("FLASHSVD_REFERENCE", ""))
    args = ap.parse_args()
    sys.path.insert(0, str(Path(args.reference).resolve()))
    from scripts.demo_support import api   # the reference's module

    cases = []
    for seed, vocab, temperature, top_p, do_sample in ((0, 50, 0.8, 0.95, True), (1, 50, 1.3, 0.5, True), (2, 7, 0.7, 1.0, True),
                                                         (3, 50, 0.0, 0.9, True), (4, 50, 0.8, 0.95, False), (5, 300, 0.5, 0.1, True),
                                                         (6, 12, 2.0, 0.999, True)):
        logits = torch.randn(3, vocab, generator=torch.Generator().manual_seed(100 + seed)) * 3.0
        torch.manual_seed(seed)
        draws = [api._sample_next_token(logits, do_sample=do_sample, temperature=temperature, top_p=top_p).view(-1).tolist()
                 for _ in range(6)]
        cases.append({"seed": seed, "vocab": vocab, "temperature": temperature, "top_p": top_p, "do_sample": do_sample,
                      "draws": draws})
    OUT.write_text(json.dumps(cases, indent=1) + "\n")
    print(f"wrote {OUT}")


if __name__ == "__main__":
    main()
