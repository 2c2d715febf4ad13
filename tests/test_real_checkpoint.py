"""Integration with a real checkpoint directory, when one is given (``CUBIC_REAL_CHECKPOINT=/path``): admission under the
closed inventory, a few greedy tokens on the eager model of its family, and (on a GPU) native logits against the eager
model's.  Skipped otherwise: no checkpoint ships with the repository."""
import os

import pytest
import torch

PATH = os.environ.get("CUBIC_REAL_CHECKPOINT")
needs_checkpoint = pytest.mark.skipif(not PATH, reason="set CUBIC_REAL_CHECKPOINT to a checkpoint directory")


def _eager_model(ck):
    from cubic_serve_b200.models import eager_family as EF
    return EF.EagerFamilyModel(ck.cfg, EF.family_weights_from_checkpoint(ck), kv_bits=(8, 8))


@needs_checkpoint
def test_admission_and_eager_tokens():
    from cubic_serve_b200.models.checkpoint import admit_checkpoint, inspect_checkpoint
    info = inspect_checkpoint(PATH)
    assert info["tensors"] > 0
    ck = admit_checkpoint(PATH)
    model = _eager_model(ck)
    prompt = [t % ck.cfg.vocab_size for t in range(11, 43)]
    logits, state = model.forward(prompt, last_only=True)
    out = []
    for _ in range(4):
        out.append(int(logits[0].argmax()))
        logits, state = model.forward([out[-1]], state, last_only=True)
    assert len(out) == 4 and bool(torch.isfinite(logits).all())
    again, _ = model.forward(prompt, last_only=True)
    assert int(again[0].argmax()) == out[0]


@needs_checkpoint
@pytest.mark.gpu
def test_native_logits_against_the_eager_model():
    from cubic_serve_b200.models.checkpoint import admit_checkpoint, load_decoder_weights
    from cubic_serve_b200.parallel.tp_check import _rel_rows, _step_logits
    ck = admit_checkpoint(PATH)
    dev = torch.device("cuda")
    prompts = [[(7 * i + 3 * j) % ck.cfg.vocab_size for j in range(48)] for i in range(4)]
    (l0, _), _ = _step_logits(ck.cfg, load_decoder_weights(ck, dev), dev, None, prompts, 8, 8)
    model = _eager_model(ck)
    want = torch.stack([model.forward(p, last_only=True)[0][0] for p in prompts])
    err = _rel_rows(l0.cpu(), want)
    assert float(err.median()) < 0.08, err
