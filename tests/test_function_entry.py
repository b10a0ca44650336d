"""A model function compiled as an inference entry (compile::compile_function,
crates/modelspec-core/src/compile.rs:173-288; the cases of its unit tests :733-810): one input
per argument, the function's result the prediction, its mean (or the rank-0 result itself) the
loss, sgd whatever the block's optimizer, every dropout the identity, and E-DATA-010 naming the
model's functions for a name it does not declare. No GPU."""
import pytest

import modelspec_b200 as M

SEVERAL = """model Several {
    param w: Tensor<f32, [3, 2]> = xavier_uniform();
    param b: Tensor<f32, [2]> = zeros();

    fn forward(x: Tensor<f32, [4, 3]>, y: Tensor<f32, [4, 2]>) -> Tensor<f32, []> {
        return mse(scores(x), y);
    }

    fn scores(x: Tensor<f32, [4, 3]>) -> Tensor<f32, [4, 2]> {
        return add_rows(matmul(x, w), b);
    }

    fn picked(table: Tensor<f32, [6, 3]>, ids: Tensor<i32, [4]>) -> Tensor<f32, [4, 3]> {
        return embedding(table, ids);
    }

    fn noisy(x: Tensor<f32, [4, 3]>) -> Tensor<f32, [4, 2]> {
        return dropout(matmul(x, w), p = 0.5);
    }
}
train Fit {
    model = Several;
    input x: Tensor<f32, [4, 3]>;
    target y: Tensor<f32, [4, 2]>;
    loss = model.forward(x, y);
    optimizer = adamw(lr = 0.1, weight_decay = 0.01, beta1 = 0.9, beta2 = 0.999, eps = 1e-8, warmup_steps = 1);
    steps = 3;
    seed = 5;
    device = cpu;
}
"""


def inputs_of(text):
    return [line.split('Input "')[1].split('"')[0] for line in text.splitlines() if '= Input "' in line]


def node(text, value):
    """The line that defines `%n`."""
    for line in text.splitlines():
        if line.strip().startswith(value + ":"):
            return line
    raise AssertionError("%s is not defined in\n%s" % (value, text))


def test_a_named_function_has_its_arguments_as_inputs_and_its_result_predicted():
    forward = M.compile_function(SEVERAL, "scores", "forward")
    assert inputs_of(forward) == ["x"]
    prediction = M.compile_function(SEVERAL, "scores", "prediction")
    assert "Tensor<f32, [4, 2]> = AddRows" in node(forward, prediction)
    # the loss is the mean of the result, and the program's one output
    means = [l for l in forward.splitlines() if "= ReduceMean " in l]
    assert len(means) == 1 and means[0].rstrip().endswith("ReduceMean " + prediction)
    # sgd whatever the block's optimizer, on the file's parameter table
    step = M.compile_function(SEVERAL, "scores", "step")
    assert any(l.startswith("optimizer sgd lr = 0.1") for l in step.splitlines()) and "adamw" not in step
    file_params = [l for l in M.compile_mspec(SEVERAL, "forward").splitlines() if l.startswith("param ")]
    assert [l for l in forward.splitlines() if l.startswith("param ")] == file_params and len(file_params) == 2


def test_forward_itself_is_an_entry_whose_result_is_the_loss():
    forward = M.compile_function(SEVERAL, "forward", "forward")
    assert inputs_of(forward) == ["x", "y"]
    prediction = M.compile_function(SEVERAL, "forward", "prediction")
    assert "Tensor<f32, []> = Mse" in node(forward, prediction) and "ReduceMean" not in forward
    outputs = [l for l in forward.splitlines() if l.startswith("output")]
    assert len(outputs) == 1 and prediction in outputs[0]


def test_a_function_without_parameters_and_one_with_dropout_compile():
    picked = M.compile_function(SEVERAL, "picked", "forward")
    assert inputs_of(picked) == ["table", "ids"] and "ParamRead" not in picked
    noisy = M.compile_function(SEVERAL, "noisy", "forward")
    assert inputs_of(noisy) == ["x"] and "Dropout" not in noisy
    assert "Dropout" not in M.compile_function(SEVERAL, "noisy", "step")
    assert "= MatMul" in node(noisy, M.compile_function(SEVERAL, "noisy", "prediction"))


def test_an_unknown_function_names_the_functions_of_the_model():
    with pytest.raises(M.MsxError) as e:
        M.compile_function(SEVERAL, "logits")
    message = str(e.value)
    assert "E-DATA-010: the model declares no function `logits`" in message
    assert "functions: forward, scores, picked, noisy" in message
    with pytest.raises(M.MsxError):
        M.compile_function(SEVERAL.replace("matmul(x, w), b)", "matmul(w, x), b)"), "scores")


def test_every_entry_schedules_in_f32_and_what_has_no_bf16_form_is_refused_loudly():
    for name in ("forward", "scores", "picked", "noisy"):
        for which in ("forward", "step"):
            assert "launches" in M.schedule_describe(M.compile_function(SEVERAL, name, which), M.PLAN_DEFAULT)
    with pytest.raises(M.MsxError) as e:
        M.schedule_describe(M.compile_function(SEVERAL, "scores", "forward"), M.PLAN_BF16)
    assert "E-TARGET-011" in str(e.value) and "has no CUDA kernel" in str(e.value)
