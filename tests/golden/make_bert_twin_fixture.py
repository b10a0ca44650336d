"""Writes tests/golden/bert_twin_torch.npz from the reference's own PyTorch restatement of the
BERT-tiny program (opponents/bert_tiny_pretrain/bert_tiny_pretrain.py of beyond10x/modelspec:
`forward` :513-522, `layer` :498-510, `attention` :481-495, `gelu` :475-478, the loss of
`train_loss` :525-529, the AdamW and LambdaLR set-up of `train` :644-648 with `schedule`
:547-556).

That module is imported as it stands; only its size constants are set to the hidden-32 twin the
parity tests train (2 layers, hidden 32, 2 heads, feed-forward 64, vocabulary 128, 8 sequences of
16 tokens), and it runs on the CPU in float64 with dropout off, so what it records is the step
the program defines, to far below the run tolerance. The fixture holds the initial parameters
(seeded numpy draws, so that it does not depend on this repository's initialisation), one
synthetic MLM batch, the hyperparameters, and for 10 AdamW steps on that batch the loss before
each update, then the loss, every parameter and every parameter's gradient after the last one.
Some key positions of two sequences are masked out so that the masked-softmax path is in it.

    python tests/golden/make_bert_twin_fixture.py <reference checkout>

The committed .npz is what travels; the tests never import the reference.
"""
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from modelspec_b200 import synthetic  # noqa: E402

TWIN = dict(BATCH=8, SEQ=16, HIDDEN=32, HEADS=2, FFN=64, VOCAB=128, LAYERS=2)
STEPS, WARMUP, LR = 10, 3, 3e-3


def main():
    if len(sys.argv) != 2:
        raise SystemExit(__doc__)
    path = os.path.join(sys.argv[1], "opponents", "bert_tiny_pretrain", "bert_tiny_pretrain.py")
    spec = importlib.util.spec_from_file_location("reference_bert_tiny_pretrain", path)
    ref = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(ref)
    for name, value in TWIN.items():
        setattr(ref, name, value)
    ref.LR = LR

    rng = np.random.default_rng(20260101)
    initial = {}
    for name, shape in ref.shapes():
        if len(shape) == 2:
            bound = np.sqrt(6.0 / (shape[0] + shape[1]))
            value = (rng.random(shape) * 2 - 1) * bound
        elif "gamma" in name:
            value = 1.0 + 0.1 * rng.standard_normal(shape)
        else:
            value = 0.05 * rng.standard_normal(shape)
        initial[name] = value.astype(np.float32)

    batch = synthetic.mlm_batch(0, vocab=TWIN["VOCAB"], seq=TWIN["SEQ"], batch=TWIN["BATCH"], mask_id=4)
    key_mask = batch["key_mask"].reshape(TWIN["BATCH"], TWIN["SEQ"]).copy()
    key_mask[1, 11:] = 0.0
    key_mask[5, :3] = 0.0
    batch["key_mask"] = key_mask.reshape(-1)

    params = {n: torch.tensor(v, dtype=torch.float64, requires_grad=True) for n, v in initial.items()}
    ids = torch.tensor(batch["ids"], dtype=torch.long)
    positions = torch.tensor(batch["positions"], dtype=torch.long)
    labels = torch.tensor(batch["labels"], dtype=torch.long)
    weights = torch.tensor(batch["weights"], dtype=torch.float64)
    mask = torch.tensor(key_mask, dtype=torch.float64)

    def loss_of():
        nll = torch.nn.functional.cross_entropy(ref.forward(params, ids, positions, mask, False), labels, reduction="none")
        return (weights * nll).sum() / weights.sum().clamp(min=1.0)

    leaves = [params[name] for name, _ in ref.shapes()]
    optimizer = torch.optim.AdamW(leaves, lr=ref.LR, betas=ref.BETAS, eps=ref.ADAM_EPS, weight_decay=ref.WEIGHT_DECAY)
    scheduler = torch.optim.lr_scheduler.LambdaLR(optimizer, ref.schedule(WARMUP, STEPS))
    losses, first_gradients = [], {}
    for step in range(STEPS):
        optimizer.zero_grad(set_to_none=True)
        loss = loss_of()
        loss.backward()
        if step == 0:
            first_gradients = {n: params[n].grad.detach().numpy().copy() for n in params}
        losses.append(loss.item())
        optimizer.step()
        scheduler.step()
    with torch.no_grad():
        losses.append(loss_of().item())

    out = {"losses": np.array(losses, dtype=np.float64),
           "hyper": np.array([ref.LR, ref.WEIGHT_DECAY, ref.BETAS[0], ref.BETAS[1], ref.ADAM_EPS, WARMUP, STEPS], dtype=np.float64),
           "shape": np.array([TWIN[k] for k in ("BATCH", "SEQ", "HIDDEN", "HEADS", "FFN", "VOCAB", "LAYERS")], dtype=np.int64)}
    for name, value in batch.items():
        out["batch." + name] = value
    for name in initial:
        out["initial." + name] = initial[name]
        out["final." + name] = params[name].detach().numpy().astype(np.float32)
        out["gradient0." + name] = first_gradients[name].astype(np.float32)
    np.savez_compressed(os.path.join(HERE, "bert_twin_torch.npz"), **out)
    print("wrote bert_twin_torch.npz: losses", " ".join("%.6f" % l for l in losses))


if __name__ == "__main__":
    main()
