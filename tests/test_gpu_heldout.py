"""Held-out evaluation on the device against the oracle's restatement of the reference's host
tally (crates/modelspec-runtime/src/train/eval.rs:409-499): the count of correct rows exactly, the
weighted loss sum within the kernel tolerance, on the reference's own unit-test batches (NaN,
infinity, far-apart logits, zero and negative weights), on ties, on ragged widths and row
alignments, and through a BERT-shaped run whose logits are bit-for-bit the oracle's."""
import numpy as np
import pytest

import modelspec_b200 as M
import oracle_lib
from helpers import ProgramText
from modelspec_b200 import models, synthetic

pytestmark = pytest.mark.gpu


def copy_program(rows, classes):
    """logits = x + zero: the plan's output holds the input's bits (and +0 for -0)."""
    t = ProgramText()
    x = t.input("x", "f32", [rows, classes])
    z = t.input("zero", "f32", [rows, classes])
    out = t.op("Add", [rows, classes], [x, z])
    t.output(out)
    return t.text(), out


def tally_both(device, batches, classes):
    """`batches`: [(logits [rows, classes], labels, weights)]. Returns the oracle's read() and the
    device's (numerator, correct)."""
    rows = batches[0][1].size
    text, out = copy_program(rows, classes)
    plan = M.Plan(device, text, flags=M.PLAN_GUARD)
    held = M.HeldOut(plan, out, len(batches))
    cpu = oracle_lib.Tally()
    try:
        plan.set_input("zero", np.zeros(rows * classes, dtype=np.float32))
        for b, (logits, labels, weights) in enumerate(batches):
            held.targets(b, labels, weights)
            cpu.add(logits, labels, weights)
        results = []
        for _ in range(2):  # a second evaluation starts from a clean state and gives the same bits
            held.begin()
            for b, (logits, _, _) in enumerate(batches):
                plan.set_input("x", logits)
                plan.run()
                held.add(b)
            results.append(held.sums())
        assert np.float64(results[0][0]).tobytes() == np.float64(results[1][0]).tobytes() and results[0][1] == results[1][1]
        plan.check_guards()
        return cpu.read(), results[0]
    finally:
        held.destroy()
        plan.destroy()


def close(device_numerator, cpu_numerator, scale):
    if np.isnan(cpu_numerator):
        return np.isnan(device_numerator)
    return abs(device_numerator - cpu_numerator) <= 1e-5 * scale + 1e-4 * abs(cpu_numerator)


def reference_batch(v, weights, logits):
    rows = len(weights)
    values = np.array([logits(i // v, i % v) for i in range(rows * v)], dtype=np.float32)
    return values, np.array([n % v for n in range(rows)], dtype=np.int32), np.array(weights, dtype=np.float32)


def test_the_reference_unit_test_batches(device):
    v = 8
    smooth = lambda n, c: np.float32(np.float32((n * 31 + c * 17) % 23) * np.float32(0.37) - np.float32(4.0))
    plain = [reference_batch(v, [0, 0, 1, 0, 0, 0, 1, 0], smooth), reference_batch(v, [0.5, 0, 2, 0, 0, 1, 0, 3], smooth),
             reference_batch(v, [0.0] * 8, smooth)]
    cpu, (numerator, correct) = tally_both(device, plain, v)
    assert correct == cpu[4] and close(numerator, cpu[2], 8 * 4.0)
    odd = reference_batch(v, [0, 1, 0, 0, 1, 0, 0, 0], smooth)
    odd[0][2 * v + 3] = np.nan      # a row of weight 0 with a NaN: 0 x NaN reaches the sum
    cpu, (numerator, correct) = tally_both(device, [plain[0], odd], v)
    assert np.isnan(cpu[2]) and np.isnan(numerator) and correct == cpu[4]
    far = reference_batch(v, [0, 1, 0, 0, 1, 0, 0, 0], smooth)
    far[0][5 * v] = 3.0e38          # weight 0, logits so far apart that the row is not skipped
    far[0][5 * v + 5] = -3.0e38
    cpu, (numerator, correct) = tally_both(device, [far], v)
    assert correct == cpu[4] and (np.isnan(cpu[2]) and np.isnan(numerator) or close(numerator, cpu[2], 8 * 4.0))
    peaked = lambda n, c: np.float32(0.0 if c == 0 else -1000.0)
    cpu, (numerator, correct) = tally_both(device, [reference_batch(v, [-1, 0, 0], peaked)], v)
    assert np.float64(numerator).tobytes() == np.float64(cpu[2]).tobytes(), "a sum of -0 followed by rows of weight 0 is +0"


@pytest.mark.parametrize("rows,classes", [(5, 1), (7, 3), (33, 1003), (64, 4096), (19, 30522), (300, 2050)])
def test_ragged_widths_and_row_alignments(device, rows, classes):
    rng = np.random.default_rng(rows * 7919 + classes)
    batches = []
    for b in range(3):
        logits = (rng.standard_normal(rows * classes) * 3.0).astype(np.float32)
        labels = rng.integers(0, classes, rows).astype(np.int32)
        # Half the selected rows have their label as the largest logit.
        for n in range(0, rows, 2):
            logits[n * classes + labels[n]] = 40.0
        weights = (rng.random(rows) < 0.4).astype(np.float32) * rng.choice(np.array([1.0, 0.5, 2.0], dtype=np.float32), rows)
        batches.append((logits, labels, weights))
    cpu, (numerator, correct) = tally_both(device, batches, classes)
    assert correct == cpu[4]
    assert close(numerator, cpu[2], 3 * rows * np.log(classes + 1.0))


def test_a_tie_goes_to_the_lowest_class(device):
    rows, classes = 40, 517
    rng = np.random.default_rng(5)
    logits = rng.integers(-3, 4, rows * classes).astype(np.float32)  # many equal maxima per row
    labels = np.array([int(np.argmax(logits[n * classes:(n + 1) * classes])) for n in range(rows)], dtype=np.int32)
    labels[1::2] += 1  # every other row names a later class, which may tie with the first largest but never wins
    labels = np.minimum(labels, classes - 1).astype(np.int32)
    cpu, (numerator, correct) = tally_both(device, [(logits, labels, np.ones(rows, dtype=np.float32))], classes)
    assert correct == cpu[4] == rows // 2 and close(numerator, cpu[2], rows * np.log(classes))


def test_a_label_outside_the_classes_is_refused_with_the_reference_message(device):
    text, out = copy_program(4, 8)
    plan = M.Plan(device, text)
    held = M.HeldOut(plan, out, 2)
    try:
        with pytest.raises(M.MsxError) as e:
            held.targets(1, [0, 1, 8, 2], [1, 1, 1, 1])
        assert e.value.status == M.BAD_INPUT and "held-out batch 1, row 2: label 8 is not below the 8 classes" in str(e.value)
        with pytest.raises(M.MsxError):
            held.add(0)  # no evaluation begun
        held.begin()
        with pytest.raises(M.MsxError):
            held.add(1)  # its targets were refused
    finally:
        held.destroy()
        plan.destroy()


BERT = dict(name="BertTiny", hidden=32, heads=2, ffn=64, vocab=304, seq=16, batch=8, warmup_steps=1)


def heldout_batches(count):
    return [synthetic.mlm_batch(1000 + b, vocab=304, seq=16, batch=8) for b in range(count)]


@pytest.mark.parametrize("flags,exact", [(M.PLAN_EXACT_MATMUL, True), (M.PLAN_DEFAULT, False), (M.PLAN_BF16, False)])
def test_a_bert_run_evaluates_its_held_out_split(device, flags, exact):
    source = models.bert(steps=4, **BERT)
    gpu = M.Training(device, source, 64, flags)
    cpu = oracle_lib.Trainer(source, 64)
    try:
        held = heldout_batches(3)
        gpu.heldout_begin(len(held), "labels", "weights")
        for b, tensors in enumerate(held):
            for name, value in tensors.items():
                gpu.heldout_set(b, name, value)
        before = gpu.heldout_evaluate()
        losses = []
        for k in range(4):
            for name, value in synthetic.mlm_batch(k, vocab=304, seq=16, batch=8).items():
                gpu.set_input(name, value)
            gpu.step(k, 4)
            if k == 1:
                middle = gpu.heldout_evaluate()  # between two steps, as --eval-every does
            losses.append(gpu.loss())
        after = gpu.heldout_evaluate()
        assert after == gpu.heldout_evaluate(), "an evaluation changes nothing it reads"
        assert np.isfinite([before[0], middle[0], after[0]]).all() and 0.0 <= after[1] <= 1.0
        # The oracle on the parameters the device trained: every batch through the forward program,
        # its logits through the host tally.
        for i in range(len(cpu.param_paths())):
            cpu.write_param(i, gpu.step_plan.param_download(i))
        tally = oracle_lib.Tally()
        selected = 0
        for tensors in held:
            for name, value in tensors.items():
                cpu.set_input(name, value)
            tally.add(cpu.predict(8 * 16 * 304), tensors["labels"], tensors["weights"])
            selected += int((tensors["weights"] > 0).sum())
        loss, accuracy = tally.read()[:2]
        if exact:
            # Products in the oracle's own order: logits within the kernel tolerance of the
            # oracle's, so the same rows are correct and the loss is the oracle's to 1e-4.
            assert after[1].tobytes() == accuracy.tobytes()
            assert abs(float(after[0]) - float(loss)) <= 1e-5 + 1e-4 * abs(float(loss))
        else:
            tolerance = 2e-2 if flags & M.PLAN_BF16 else 1e-3
            assert abs(float(after[0]) - float(loss)) <= 1e-4 + tolerance * abs(float(loss))
            assert abs(float(after[1]) - float(accuracy)) <= 2.0 / max(selected, 1) + (0.05 if flags & M.PLAN_BF16 else 0.0)
    finally:
        gpu.destroy()


def test_evaluating_does_not_change_the_run(device):
    source = models.bert(steps=3, **BERT)
    runs = []
    for evaluate in (False, True):
        gpu = M.Training(device, source, 64)
        try:
            if evaluate:
                gpu.heldout_begin(1, "labels", "weights")
                for name, value in heldout_batches(1)[0].items():
                    gpu.heldout_set(0, name, value)
            losses = []
            for k in range(3):
                for name, value in synthetic.mlm_batch(k, vocab=304, seq=16, batch=8).items():
                    gpu.set_input(name, value)
                gpu.step(k, 3)
                if evaluate:
                    gpu.heldout_evaluate()
                losses.append(gpu.loss())
            losses.append(gpu.final_loss())
            runs.append(np.array(losses, dtype=np.float32))
        finally:
            gpu.destroy()
    assert runs[0].tobytes() == runs[1].tobytes()


def test_a_prediction_that_is_not_logits_per_label_is_refused(device):
    gpu = M.Training(device, models.linear_regression(steps=2), 0)
    try:
        with pytest.raises(M.MsxError):
            gpu.heldout_begin(1, "y", "y")
    finally:
        gpu.destroy()
