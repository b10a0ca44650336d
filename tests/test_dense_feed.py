"""The dense `--data` directory as the reference reads it (crates/modelspec-runtime/src/train/
data.rs:14-35, dense :513-577, read_files :837-876, read_tensor :1232-1290, fill_step :446-454):
host code, no GPU."""
import os

import numpy as np
import pytest

import modelspec_b200 as M


def write(directory, name, values):
    values.tofile(str(directory / name))


DECLS = [("x", "f32", "input", [4, 3]), ("ids", "i32", "input", [4]), ("y", "f32", "target", [4, 2])]


def directory_of(tmp_path, samples=10):
    r = np.random.default_rng(5)
    x = r.standard_normal((samples, 3)).astype(np.float32)
    ids = r.integers(0, 6, size=samples).astype(np.int32)
    y = r.standard_normal((samples, 2)).astype(np.float32)
    write(tmp_path, "x.f32", x)
    write(tmp_path, "ids.i32", ids)
    write(tmp_path, "y.f32", y)
    return x, ids, y


def test_batches_follow_the_sample_rule_without_and_with_an_order(tmp_path):
    x, ids, y = directory_of(tmp_path)
    d = M.Dense(tmp_path, DECLS, steps=5)
    assert (d.batch, d.samples, d.has_order) == (4, 10, False)
    for k in (0, 1, 2, 7):
        rows = [(k * 4 + i) % 10 for i in range(4)]          # (k B + i) mod N
        assert np.array_equal(d.step(0, k), x[rows].reshape(-1))
        assert np.array_equal(d.step(1, k), ids[rows])
        assert np.array_equal(d.step(2, k), y[rows].reshape(-1))
    d.close()
    order = np.array([9, 0, 3, 3, 1, 2, 8, 7, 6, 5, 4, 4, 0, 9, 2, 1, 5, 5, 5, 5, 7], dtype=np.uint32)
    write(tmp_path, "order.u32", order)
    d = M.Dense(tmp_path, DECLS, steps=5)
    assert d.has_order
    for k in (0, 3, 5, 6):                                     # positions past the end of the order wrap
        rows = [int(order[(k * 4 + i) % len(order)]) for i in range(4)]
        assert np.array_equal(d.step(0, k), x[rows].reshape(-1))
        assert np.array_equal(d.step(1, k), ids[rows])
    d.close()


def test_declarations_without_a_shared_leading_dimension_are_one_sample_a_step(tmp_path):
    write(tmp_path, "a.f32", np.arange(12, dtype=np.float32))
    write(tmp_path, "b.f32", np.arange(6, dtype=np.float32))
    d = M.Dense(tmp_path, [("a", "f32", "input", [2, 2]), ("b", "f32", "target", [2])], steps=1)
    assert (d.batch, d.samples) == (2, 6)                      # both lead with 2: B = 2, samples of 2 values and of 1
    d.close()
    d = M.Dense(tmp_path, [("a", "f32", "input", [4]), ("b", "f32", "target", [2])], steps=1)
    assert (d.batch, d.samples) == (1, 3)                      # 4 and 2 differ: B = 1, a sample is the whole tensor
    assert np.array_equal(d.step(0, 4), np.arange(4, 8, dtype=np.float32))   # step 4 -> sample 4 mod 3
    d.close()


def refused(tmp_path, decls=DECLS, steps=5):
    with pytest.raises(M.MsxError) as e:
        M.Dense(tmp_path, decls, steps)
    assert e.value.status == M.BAD_INPUT
    return str(e.value)


def test_the_refusals_of_the_files(tmp_path):
    x, ids, y = directory_of(tmp_path)
    assert "E-DATA-001" in refused(tmp_path, decls=[])
    (tmp_path / "ids.i32").unlink()
    write(tmp_path, "ids.f32", ids.astype(np.float32))
    message = refused(tmp_path)
    assert "E-DATA-007" in message and "cannot read the data file of the input `ids`" in message and "ids.f32, the file of an f32 declaration" in message
    write(tmp_path, "ids.i32", ids)
    write(tmp_path, "y.f32", y.reshape(-1)[:-1])               # 19 values, samples of 2
    assert "is not a whole number of samples" in refused(tmp_path)
    bad = y.copy()
    bad[3, 1] = np.inf
    write(tmp_path, "y.f32", bad)
    message = refused(tmp_path)
    assert "holds a value that is not finite" in message and "index 7" in message and "value inf" in message
    write(tmp_path, "y.f32", y[:8])                            # 8 samples beside 10
    message = refused(tmp_path)
    assert "do not hold the same number of samples" in message and "x 10" in message and "y 8" in message
    with open(tmp_path / "x.f32", "ab") as f:
        f.write(b"\0")
    assert "is not a whole number of f32 values" in refused(tmp_path)


def test_the_refusals_of_the_order_and_of_an_id_outside_its_table(tmp_path):
    x, ids, y = directory_of(tmp_path)
    write(tmp_path, "order.u32", np.arange(10, dtype=np.uint32))
    message = refused(tmp_path, steps=5)                       # needs 5 x 4 = 20 indices
    assert "E-DATA-008" in message and "fewer than steps · B indices" in message and "needed 20" in message
    order = np.arange(20, dtype=np.uint32) % 10
    order[13] = 10
    write(tmp_path, "order.u32", order)
    message = refused(tmp_path, steps=5)
    assert "E-DATA-008" in message and "names a sample past the end of the data" in message and "position 13" in message
    (tmp_path / "order.u32").unlink()
    d = M.Dense(tmp_path, DECLS, steps=5)
    d.check_bound(1, 6, "the 6 rows of the `embedding` table `Named.table`")   # ids are 0 .. 5
    d.check_bound(0, 1, "unused")                                                # an f32 file has no bound
    with pytest.raises(M.MsxError) as e:
        d.check_bound(1, int(ids.max()), "the %d rows of the `embedding` table `Named.table`" % ids.max())
    message = str(e.value)
    first = int(np.argmax(ids >= ids.max()))
    assert "E-DATA-011" in message and "outside the %d rows" % ids.max() in message and "position %d" % first in message
    d.close()


def test_an_eval_directory_is_whole_batches_and_reads_no_order(tmp_path):
    x, ids, y = directory_of(tmp_path, samples=12)
    write(tmp_path, "order.u32", np.array([99], dtype=np.uint32))   # would be refused by a --data directory; --eval does not read it
    d = M.Dense(tmp_path, DECLS, steps=0, eval_directory=True)
    assert (d.batch, d.samples, d.has_order) == (4, 12, False)
    for b in range(3):
        assert np.array_equal(d.eval_batch(0, b), x[4 * b:4 * b + 4].reshape(-1))
        assert np.array_equal(d.eval_batch(1, b), ids[4 * b:4 * b + 4])
    with pytest.raises(M.MsxError):
        d.eval_batch(0, 3)
    d.close()
    directory_of(tmp_path, samples=10)
    with pytest.raises(M.MsxError) as e:
        M.Dense(tmp_path, DECLS, steps=0, eval_directory=True)
    message = str(e.value)
    assert "E-DATA-009" in message and "not a whole number of batches" in message and "samples 10" in message and "batch 4" in message


def test_the_arguments_of_a_function_are_named_so_and_come_in_whole_blocks(tmp_path):
    """dense_function (train/data.rs:685-717): the files of a function's arguments are read as an
    eval directory's, the messages say `argument`, and E-DATA-009 speaks of blocks."""
    arguments = [(name, dtype, "argument", shape) for name, dtype, _, shape in DECLS]
    x, ids, y = directory_of(tmp_path, samples=8)
    d = M.Dense(tmp_path, arguments, steps=0, eval_directory=True)
    assert (d.batch, d.samples) == (4, 8)
    with pytest.raises(M.MsxError) as e:
        d.check_bound(1, 1, "the 1 rows of the `embedding` table `%0`")
    assert "E-DATA-011: the data file of the argument `%s` holds" % arguments[1][0] in str(e.value)
    d.close()
    directory_of(tmp_path, samples=10)
    with pytest.raises(M.MsxError) as e:
        M.Dense(tmp_path, arguments, steps=0, eval_directory=True)
    assert "E-DATA-009: the data is not a whole number of blocks (directory" in str(e.value) and "samples 10, batch 4" in str(e.value)
    os.remove(os.path.join(str(tmp_path), "%s.f32" % arguments[0][0]))
    with pytest.raises(M.MsxError) as e:
        M.Dense(tmp_path, arguments, steps=0, eval_directory=True)
    assert "E-DATA-007: cannot read the data file of the argument `%s`" % arguments[0][0] in str(e.value)


def test_the_eval_line_prints_f64_as_the_reference_does():
    assert M.eval_line(0.125, 0.5) == "eval loss=0.125 accuracy=0.5\n"
    assert M.eval_line(3.0, 1.0) == "eval loss=3 accuracy=1\n"
    assert M.eval_line(1e-7) == "eval loss=0.0000001\n"
    assert M.eval_line(0.1 + 0.2) == "eval loss=0.30000000000000004\n"
