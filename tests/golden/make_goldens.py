"""Writes the fixtures of tests/golden/ from a checkout of the reference (beyond10x/modelspec).

The fixtures are the reference's own recorded outputs for this path, reduced to the numbers the
tests compare: the per-step losses of two recorded CPU runs
(crates/modelspec-cli/tests/fixtures/{linear_regression,two_layer_relu}.run.jsonl), the initial
and final parameter of the linear-regression training log
(crates/modelspec-cli/tests/golden/linear_regression.train.stdout), the printed training IR of
two examples (crates/modelspec-cli/tests/golden/*.training.ir) and the lowered BERT-tiny program
(website/docs/examples/bert-tiny.md). BLAKE3 digests come from the `blake3` Python package.
Run it where the reference is checked out (the committed fixtures are what travels):
`python tests/golden/make_goldens.py <reference checkout>`.
"""
import json
import os
import re
import sys

if len(sys.argv) != 2:
    raise SystemExit(__doc__)
REF = sys.argv[1]
HERE = os.path.dirname(os.path.abspath(__file__))


def losses(path):
    out = []
    for line in open(path):
        event = json.loads(line)
        if event["body"]["kind"] == "StepCompleted":
            out.append(event["body"]["value"]["loss"])
    return out


def vector(line):
    return [float(x) for x in re.search(r"\[([^\]]*)\]$", line.strip()).group(1).split(",")]


def main():
    fixtures = os.path.join(REF, "crates/modelspec-cli/tests/fixtures")
    golden = os.path.join(REF, "crates/modelspec-cli/tests/golden")
    log = open(os.path.join(golden, "linear_regression.train.stdout")).read().splitlines()
    json.dump({"losses": losses(os.path.join(fixtures, "linear_regression.run.jsonl")),
               "initial_param": vector(log[0]), "final_param": vector(log[-1]),
               "log": log},
              open(os.path.join(HERE, "linear_regression.losses.json"), "w"))
    json.dump({"losses": losses(os.path.join(fixtures, "two_layer_relu.run.jsonl"))},
              open(os.path.join(HERE, "two_layer_relu.losses.json"), "w"))
    for name in ("linear_regression.training.ir", "linear_regression.tensor.ir", "mnist_mlp.training.ir"):
        open(os.path.join(HERE, name), "w").write(open(os.path.join(golden, name)).read())
    doc = open(os.path.join(REF, "website/docs/examples/bert-tiny.md")).read()
    block = doc.split("### `modelspec ir examples/bert_tiny.mspec --stage tensor`")[1].split("```text", 1)[1].split("```")[0].lstrip("\r\n")
    open(os.path.join(HERE, "bert_tiny.tensor.ir"), "w").write(block)
    import blake3
    cases = {}
    for n in (0, 1, 3, 63, 64, 65, 127, 128, 1023, 1024, 1025, 2048, 2049, 3072, 5000):
        data = bytes((i * 7 + 3) % 251 for i in range(n))
        cases[str(n)] = blake3.blake3(data).hexdigest()
    cases["path:LinearReg.w"] = blake3.blake3(b"LinearReg.w").hexdigest()
    json.dump(cases, open(os.path.join(HERE, "blake3.json"), "w"), indent=0)


if __name__ == "__main__":
    main()
