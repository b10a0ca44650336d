"""Child process of the fusion A/B test: trains the hidden-32 BERT twin for a few steps under the
MSX_FUSE mask of its environment (the mask is read once per process) and prints the bits of every
loss and a digest of every parameter, for f32 and mixed-precision plans."""
import hashlib
import json
import sys

import numpy as np

import modelspec_b200 as M
from modelspec_b200 import models, synthetic


def main():
    steps = 4
    source = models.bert(name="BertTiny", hidden=64, heads=2, ffn=128, vocab=304, seq=16, batch=8, warmup_steps=1, steps=steps)
    device = M.Device(0)
    out = {}
    for name, flags in (("f32", M.PLAN_DEFAULT), ("bf16", M.PLAN_BF16)):
        gpu = M.Training(device, source, 64, flags)
        losses = []
        for k in range(steps):
            for key, value in synthetic.mlm_batch(k, vocab=304, seq=16, batch=8).items():
                gpu.set_input(key, value)
            gpu.step(k, steps)
            losses.append(int(np.float32(gpu.loss()).view(np.uint32)))
        digest = hashlib.sha256()
        ckpt = gpu.checkpoint(steps)
        digest.update(ckpt.encode())
        ckpt.destroy()
        out[name] = {"losses": losses, "state": digest.hexdigest(), "launches": gpu.step_plan.stats()["launches_per_step"],
                     "listing_names_bits": "scratch" in gpu.step_plan.describe()}
        gpu.destroy()
    print(json.dumps(out))


if __name__ == "__main__":
    sys.exit(main())
