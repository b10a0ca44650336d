"""The oracle's held-out tally against the cases the reference's own unit tests hold it to
(crates/modelspec-runtime/src/train/eval.rs:507-633): the tally that skips the softmax of rows
that cannot change its sums gives the bits of the one that computes every row, takes exactly the
softmaxes the reference counts, a row of equal logits has the loss ln V, and a tie goes to the
lowest class."""
import numpy as np

import oracle_lib


def batch(v, weights, logits):
    rows = len(weights)
    values = np.array([logits(i // v, i % v) for i in range(rows * v)], dtype=np.float32)
    return values, np.array([n % v for n in range(rows)], dtype=np.int32), np.array(weights, dtype=np.float32)


def both(batches):
    out = []
    for skipping in (True, False):
        tally = oracle_lib.Tally(skipping)
        for logits, labels, weights in batches:
            tally.add(logits, labels, weights)
        out.append(tally.read())
    return out


def smooth(a, b, m, scale, shift):
    return lambda n, c: np.float32(np.float32((n * a + c * b) % m) * np.float32(scale) - np.float32(shift))


def test_a_row_of_equal_logits_has_the_loss_ln_v():
    tally = oracle_lib.Tally(False)
    tally.add(np.zeros(4, dtype=np.float32), [2], [1.0])
    assert tally.read()[0] == np.log(np.float32(4.0))


def test_only_the_rows_that_can_change_the_sums_take_a_softmax():
    v = 8
    f = smooth(31, 17, 23, 0.37, 4.0)
    odd = batch(v, [0, 1, 0, 0, 1, 0, 0, 0], f)
    odd[0][2 * v + 3] = np.nan
    odd[0][3 * v + 1] = np.inf
    odd[0][5 * v] = 3.0e38
    odd[0][5 * v + 5] = -3.0e38
    batches = [batch(v, [0, 0, 1, 0, 0, 0, 1, 0], f), odd, batch(v, [0.0] * 8, f)]
    skipped, every = both(batches)
    assert skipped[6] == 2 + 2 + 3 and every[6] == 24
    assert skipped[0].tobytes() == every[0].tobytes() and skipped[1].tobytes() == every[1].tobytes()


def test_skipping_a_row_keeps_the_bits_of_every_sum():
    v = 8
    f = smooth(13, 7, 19, 0.81, 6.0)
    peaked = lambda n, c: np.float32(0.0 if c == 0 else -1000.0)
    cases = [[batch(v, [0, 1, 0, 1], f)], [batch(v, [-1, 0, 0], peaked)], [batch(v, [0, 0, 0], f)],
             [batch(v, [0.5, 0, 2, 0, 0, 1], f), batch(v, [0, 0, 1, 0, 3, 0], peaked)]]
    for batches in cases:
        skipped, every = both(batches)
        assert skipped[0].tobytes() == every[0].tobytes() and skipped[1].tobytes() == every[1].tobytes()
        assert np.float64(skipped[2]).tobytes() == np.float64(every[2]).tobytes(), "the numerator keeps its sign of zero too"


def test_a_tie_goes_to_the_lowest_class_and_a_nan_row_is_never_correct():
    tally = oracle_lib.Tally()
    tally.add(np.array([1, 3, 3, 2, 1, np.nan, 0, 0], dtype=np.float32), [1, 0], [1.0, 1.0])
    assert tally.read()[4:6] == (1, 2)
    other = oracle_lib.Tally()
    other.add(np.array([1, 3, 3, 2], dtype=np.float32), [2], [1.0])
    assert other.read()[4:6] == (0, 1)
