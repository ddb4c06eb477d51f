"""The plain implementation against ling0322/libllm's own CPU code on two tiny random models.

tests/golden/*.npz were made by tests/golden/make_golden.py, which compiles the
reference's unmodified CPU sources and runs its LlamaModel (float32 arithmetic on
weights and a cos/sin table rounded to float16).  The plain implementation gets the
same rounded weights and the same table here, so what is compared is every formula
of the model except the rotary frequencies, which the reference does not compute."""
import os
import sys

import numpy as np
import pytest
import torch

import plain_llama as P

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden"))
import cases  # noqa: E402

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.mark.parametrize("name", sorted(cases.CASES))
def test_plain_implementation_matches_the_reference_cpu_code(name):
    case = cases.CASES[name]
    gold = np.load(os.path.join(GOLDEN, f"{name}.npz"))
    # the weights the reference ran with lie in the file (float16, its tensor file's precision), so
    # the comparison does not hinge on this numpy drawing the same numbers again
    w = {k[2:]: torch.from_numpy(gold[k].astype(np.float32)) for k in gold.files if k.startswith("w/")}
    assert cases.checksum(w) == str(gold["checksum"])
    c = dict(case["config"])
    c["rope_table"] = cases.rope_table(c)
    logits = P.forward_logits(c, w, case["ids"])
    ref = torch.from_numpy(gold["logits"]).double()
    got = logits[torch.tensor(gold["rows"])]
    scale = float(ref.abs().mean())
    # the reference adds in float32 (rounding 6e-8 relative, a few hundred terms per sum)
    assert float((got - ref).abs().max()) < 2e-5 * scale
    assert torch.equal(got.argmax(-1), ref.argmax(-1))
    # its token-by-token path agrees with its whole-prompt path, and so with the plain implementation
    last = torch.from_numpy(gold["last_token_by_token"]).double()
    assert float((logits[-1] - last).abs().max()) < 2e-5 * scale
