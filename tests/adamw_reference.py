"""The reference's own written-order AdamW and SGD updates, transcribed as numpy float32
arithmetic: a second restatement, independent of the oracle's and of the CUDA kernel's.

Follows crates/modelspec-runtime/tests/adamw.rs of the reference: `settled` (:118-125),
`host_constants` (:134-141), `reference` (:145-165) and the dense fixture of
`zero_gradient_decays_the_moments` (`zero_step_data`, :238-262). Every elementwise operation is one
rounded f32 operation in the written order; `lr_t`, `c1`, `c2` and each `1 - beta` are computed in
f64 and rounded once. numpy's float32 `+ - * /` and `sqrt` round once, like Rust's.
"""
import numpy as np

F = np.float32


def powi(x, n):
    """x^n by repeated squaring, as Rust's f64::powi multiplies it out."""
    r = 1.0
    while True:
        if n & 1:
            r *= x
        n >>= 1
        if n == 0:
            return r
        x *= x


def settled(lr, t, warmup_steps, steps):
    lr = float(F(lr))
    if t <= warmup_steps:
        return lr * float(t) / float(warmup_steps)
    return lr * float(steps - t) / float(steps - warmup_steps)


def host_constants(lr, beta1, beta2, t, warmup_steps, steps):
    correction = lambda beta: F(1.0 / (1.0 - powi(float(F(beta)), t)))
    return F(settled(lr, t, warmup_steps, steps)), correction(beta1), correction(beta2)


def adamw_step(p, g, m, v, constants, beta1, beta2, eps, weight_decay):
    """One update of float32 arrays; returns (p', m', v')."""
    lr_t, c1, c2 = (F(c) for c in constants)
    beta1, beta2, eps, weight_decay = F(beta1), F(beta2), F(eps), F(weight_decay)
    rest1 = F(1.0 - float(beta1))
    rest2 = F(1.0 - float(beta2))
    p, g, m, v = (np.asarray(a, dtype=F) for a in (p, g, m, v))
    decayed_m = beta1 * m
    new_m = rest1 * g
    m = decayed_m + new_m
    decayed_v = beta2 * v
    scaled_g = rest2 * g
    new_v = scaled_g * g
    v = decayed_v + new_v
    m_hat = m * c1
    v_hat = v * c2
    root = np.sqrt(v_hat)
    denominator = root + eps
    direction = m_hat / denominator
    shrink = weight_decay * p
    step = direction + shrink
    scaled = lr_t * step
    return p - scaled, m, v


def sgd_step(p, g, lr):
    """p - f32(lr * g) (attach_sgd, crates/modelspec-core/src/ir/training.rs:737-797)."""
    return np.asarray(p, dtype=F) - F(lr) * np.asarray(g, dtype=F)


# The hyperparameters and the source of the reference's AdamW tests (adamw.rs:33-63).
LR, WEIGHT_DECAY, BETA1, BETA2, EPS = 0.01, 0.1, 0.9, 0.999, 1e-8
ZERO_STEP, DENSE_STEPS = 3, 6


def two_parameters(warmup_steps, steps, rows=8, inputs=4, outputs=1):
    return """model Reg {
    param w: Tensor<f32, [%(i)d, %(o)d]> = xavier_uniform();
    param b: Tensor<f32, [%(o)d]> = zeros();

    fn forward(x: Tensor<f32, [%(r)d, %(i)d]>) -> Tensor<f32, [%(r)d, %(o)d]> {
        return add_rows(matmul(x, w), b);
    }
}

train Fit {
    model = Reg;
    input x: Tensor<f32, [%(r)d, %(i)d]>;
    target y: Tensor<f32, [%(r)d, %(o)d]>;
    loss = mse(model.forward(x), y);
    optimizer = adamw(lr = 0.01, weight_decay = 0.1, beta1 = 0.9, beta2 = 0.999, eps = 1e-8, warmup_steps = %(w)d);
    steps = %(s)d;
    seed = 7;
    device = cpu;
}
""" % {"r": rows, "i": inputs, "o": outputs, "w": warmup_steps, "s": steps}


def zero_step_batches():
    """One batch of 8 samples per step of a 6-step run; the input of step 3 is all zero."""
    samples = 8 * DENSE_STEPS
    x = np.array([0.0 if (k // 4) // 8 == ZERO_STEP else (float(k * 7 % 11) - 5.0) / 4.0 for k in range(samples * 4)], dtype=F)
    y = np.array([float(k % 5) * 0.5 - 1.0 for k in range(samples)], dtype=F)
    return [{"x": x[s * 32:(s + 1) * 32], "y": y[s * 8:(s + 1) * 8]} for s in range(DENSE_STEPS)]
