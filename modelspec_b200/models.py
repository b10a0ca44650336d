"""`.mspec` source text of the models this backend is measured and tested on.

The reference's front door reads a model as `.mspec` source (examples/*.mspec); these functions
write such source for the benchmark configurations (MLP classifier, one post-LN encoder block,
BERT-shaped MLM models) and for the small models whose recorded outputs pin the oracle. Parameter
names follow the reference's examples (`l0_wq`, `mlm_bias`, ...): a parameter's initial values are
addressed by the hash of its canonical path, so the names are part of the numbers.
"""


def _tensor(dtype, shape):
    return "Tensor<%s, [%s]>" % (dtype, ", ".join(str(d) for d in shape))


def _fmt(x):
    return repr(float(x)) if not isinstance(x, str) else x


def optimizer_line(kind, lr, weight_decay=0.01, beta1=0.9, beta2=0.999, eps=1e-8, warmup_steps=0):
    if kind == "sgd":
        return "sgd(lr = %s)" % _fmt(lr)
    return ("adamw(lr = %s, weight_decay = %s, beta1 = %s, beta2 = %s, eps = %s, warmup_steps = %d)"
            % (_fmt(lr), _fmt(weight_decay), _fmt(beta1), _fmt(beta2), _fmt(eps), warmup_steps))


def linear_regression(steps=500, seed=42):
    """8 x 4 inputs, one [4, 1] weight, MSE, SGD lr 0.1: the reference's smallest example."""
    return """model LinearReg {
    param w: Tensor<f32, [4, 1]> = xavier_uniform();
    fn forward(x: Tensor<f32, [8, 4]>) -> Tensor<f32, [8, 1]> {
        return matmul(x, w);
    }
}
train Fit {
    model = LinearReg;
    input x: Tensor<f32, [8, 4]>;
    target y: Tensor<f32, [8, 1]>;
    loss = mse(model.forward(x), y);
    optimizer = sgd(lr = 0.1);
    steps = %d;
    seed = %d;
    device = cpu;
}
""" % (steps, seed)


def two_layer_relu(steps=200, seed=7):
    return """model TwoLayer {
    param w1: Tensor<f32, [4, 8]> = xavier_uniform();
    param w2: Tensor<f32, [8, 1]> = xavier_uniform();
    fn forward(x: Tensor<f32, [16, 4]>) -> Tensor<f32, [16, 1]> {
        let h = relu(matmul(x, w1));
        return matmul(h, w2);
    }
}
train FitTwoLayer {
    model = TwoLayer;
    input x: Tensor<f32, [16, 4]>;
    target y: Tensor<f32, [16, 1]>;
    loss = mse(model.forward(x), y);
    optimizer = sgd(lr = 0.05);
    steps = %d;
    seed = %d;
    device = cpu;
}
""" % (steps, seed)


def mnist_mlp(batch=100, hidden=64, steps=1800, seed=42):
    """784 -> hidden relu -> 10, no bias, MSE, SGD: the shapes of the reference's MNIST example."""
    return """model MnistMlp {
    param w1: Tensor<f32, [784, %(h)d]> = xavier_uniform();
    param w2: Tensor<f32, [%(h)d, 10]> = xavier_uniform();
    fn forward(x: Tensor<f32, [%(b)d, 784]>) -> Tensor<f32, [%(b)d, 10]> {
        return matmul(relu(matmul(x, w1)), w2);
    }
}
train Fit {
    model = MnistMlp;
    input x: Tensor<f32, [%(b)d, 784]>;
    target y: Tensor<f32, [%(b)d, 10]>;
    loss = mse(model.forward(x), y);
    optimizer = sgd(lr = 0.1);
    steps = %(s)d;
    seed = %(seed)d;
    device = cpu;
}
""" % {"b": batch, "h": hidden, "s": steps, "seed": seed}


def mlp_classifier(batch=64, inputs=784, hidden=128, classes=10, lr=0.1, steps=500, seed=42):
    """The MLP classifier configuration: inputs -> hidden relu -> classes with biases, softmax
    cross-entropy on integer labels with unit weights, SGD."""
    return """model Mlp {
    param w1: Tensor<f32, [%(i)d, %(h)d]> = xavier_uniform();
    param b1: Tensor<f32, [%(h)d]> = zeros();
    param w2: Tensor<f32, [%(h)d, %(c)d]> = xavier_uniform();
    param b2: Tensor<f32, [%(c)d]> = zeros();
    fn forward(x: Tensor<f32, [%(b)d, %(i)d]>) -> Tensor<f32, [%(b)d, %(c)d]> {
        let h = relu(add_rows(matmul(x, w1), b1));
        return add_rows(matmul(h, w2), b2);
    }
}
train Classify {
    model = Mlp;
    input x: Tensor<f32, [%(b)d, %(i)d]>;
    target labels: Tensor<i32, [%(b)d]>;
    target weights: Tensor<f32, [%(b)d]>;
    loss = cross_entropy(model.forward(x), labels, weights);
    optimizer = sgd(lr = %(lr)s);
    steps = %(s)d;
    seed = %(seed)d;
    device = cpu;
}
""" % {"b": batch, "i": inputs, "h": hidden, "c": classes, "lr": _fmt(lr), "s": steps, "seed": seed}


def _encoder_params(layer, hidden, ffn):
    p = "l%d_" % layer
    lines = []
    for w in ("q", "k", "v", "o"):
        lines.append("    param %sw%s: %s = xavier_uniform();" % (p, w, _tensor("f32", [hidden, hidden])))
        lines.append("    param %sb%s: %s = zeros();" % (p, w, _tensor("f32", [hidden])))
    lines.append("    param %sln1_gamma: %s = ones();" % (p, _tensor("f32", [hidden])))
    lines.append("    param %sln1_beta: %s = zeros();" % (p, _tensor("f32", [hidden])))
    lines.append("    param %sw1: %s = xavier_uniform();" % (p, _tensor("f32", [hidden, ffn])))
    lines.append("    param %sb1: %s = zeros();" % (p, _tensor("f32", [ffn])))
    lines.append("    param %sw2: %s = xavier_uniform();" % (p, _tensor("f32", [ffn, hidden])))
    lines.append("    param %sb2: %s = zeros();" % (p, _tensor("f32", [hidden])))
    lines.append("    param %sln2_gamma: %s = ones();" % (p, _tensor("f32", [hidden])))
    lines.append("    param %sln2_beta: %s = zeros();" % (p, _tensor("f32", [hidden])))
    return lines


def _encoder_body(layer, x, heads, dropout):
    """Post-layer-norm encoder layer reading `x`; returns its lines and the name of its output."""
    p = "l%d_" % layer
    i = layer

    def drop(e):
        return "dropout(%s, p = %s)" % (e, _fmt(dropout)) if dropout > 0 else e

    lines = [
        "        let q%d = add_rows(matmul(%s, %swq), %sbq);" % (i, x, p, p),
        "        let k%d = add_rows(matmul(%s, %swk), %sbk);" % (i, x, p, p),
        "        let v%d = add_rows(matmul(%s, %swv), %sbv);" % (i, x, p, p),
        "        let a%d = add_rows(matmul(attention(q%d, k%d, v%d, key_mask, heads = %d), %swo), %sbo);"
        % (i, i, i, i, heads, p, p),
        "        let h%d = layer_norm(add(%s, %s), %sln1_gamma, %sln1_beta);" % (i, x, drop("a%d" % i), p, p),
        "        let f%d = add_rows(matmul(gelu(add_rows(matmul(h%d, %sw1), %sb1)), %sw2), %sb2);" % (i, i, p, p, p, p),
        "        let x%d = layer_norm(add(h%d, %s), %sln2_gamma, %sln2_beta);" % (i, i, drop("f%d" % i), p, p),
    ]
    return lines, "x%d" % i


def transformer_block(batch=8, seq=128, hidden=128, heads=2, ffn=512, layers=2, dropout=0.0,
                      optimizer="sgd", lr=0.01, steps=100, seed=42, **adamw):
    """Post-LN encoder layers on an activation input with an MSE loss. The defaults are the
    reference's transformer-block benchmark (two layers, SGD, no dropout, 8 sequences)."""
    rows = batch * seq
    lines = ["model TransformerBlock {"]
    for layer in range(layers):
        lines += _encoder_params(layer, hidden, ffn)
    xt = _tensor("f32", [rows, hidden])
    lines.append("    fn forward(x: %s, key_mask: %s) -> %s {" % (xt, _tensor("f32", [batch, seq]), xt))
    x = "x"
    for layer in range(layers):
        body, x = _encoder_body(layer, x, heads, dropout)
        if layer == layers - 1:
            # The last layer's output is the return value, not a let.
            lines += body[:-1]
            lines.append("        return " + body[-1].split(" = ", 1)[1])
        else:
            lines += body
    lines += ["    }", "}", "train Fit {", "    model = TransformerBlock;",
              "    input x: %s;" % xt, "    input key_mask: %s;" % _tensor("f32", [batch, seq]),
              "    target y: %s;" % xt, "    loss = mse(model.forward(x, key_mask), y);",
              "    optimizer = %s;" % optimizer_line(optimizer, lr, **adamw),
              "    steps = %d;" % steps, "    seed = %d;" % seed, "    device = cpu;", "}"]
    return "\n".join(lines) + "\n"


def bert(name="BertTiny", layers=2, hidden=128, heads=2, ffn=512, vocab=30522, seq=128, batch=32,
         dropout=0.1, lr=1e-4, weight_decay=0.01, beta1=0.9, beta2=0.999, eps=1e-6, warmup_steps=10,
         steps=100, seed=42):
    """A BERT-shaped masked-language model: token and learned position embeddings, post-LN
    encoder layers, an MLM head whose decoder is the token table transposed with its own bias,
    weighted cross-entropy, AdamW. The defaults are BERT-tiny at BERT's vocabulary."""
    rows = batch * seq
    lines = ["model %s {" % name,
             "    param tok_table: %s = xavier_uniform();" % _tensor("f32", [vocab, hidden]),
             "    param pos_table: %s = xavier_uniform();" % _tensor("f32", [seq, hidden]),
             "    param emb_ln_gamma: %s = ones();" % _tensor("f32", [hidden]),
             "    param emb_ln_beta: %s = zeros();" % _tensor("f32", [hidden])]
    for layer in range(layers):
        lines += _encoder_params(layer, hidden, ffn)
    lines += ["    param mlm_w: %s = xavier_uniform();" % _tensor("f32", [hidden, hidden]),
              "    param mlm_b: %s = zeros();" % _tensor("f32", [hidden]),
              "    param mlm_ln_gamma: %s = ones();" % _tensor("f32", [hidden]),
              "    param mlm_ln_beta: %s = zeros();" % _tensor("f32", [hidden]),
              "    param mlm_bias: %s = zeros();" % _tensor("f32", [vocab])]
    ids_t, mask_t = _tensor("i32", [rows]), _tensor("f32", [batch, seq])
    lines.append("    fn forward(ids: %s, positions: %s, key_mask: %s) -> %s {"
                 % (ids_t, ids_t, mask_t, _tensor("f32", [rows, vocab])))
    emb = "layer_norm(add(embedding(tok_table, ids), embedding(pos_table, positions)), emb_ln_gamma, emb_ln_beta)"
    lines.append("        let e = %s;" % ("dropout(%s, p = %s)" % (emb, _fmt(dropout)) if dropout > 0 else emb))
    x = "e"
    for layer in range(layers):
        body, x = _encoder_body(layer, x, heads, dropout)
        lines += body
    lines += ["        let m = layer_norm(gelu(add_rows(matmul(%s, mlm_w), mlm_b)), mlm_ln_gamma, mlm_ln_beta);" % x,
              "        return add_rows(matmul(m, transpose(tok_table)), mlm_bias);", "    }", "}",
              "train Pretrain {", "    model = %s;" % name,
              "    input ids: %s;" % ids_t, "    input positions: %s;" % ids_t, "    input key_mask: %s;" % mask_t,
              "    target labels: %s;" % ids_t, "    target weights: %s;" % _tensor("f32", [rows]),
              "    loss = cross_entropy(model.forward(ids, positions, key_mask), labels, weights);",
              "    optimizer = %s;" % optimizer_line("adamw", lr, weight_decay, beta1, beta2, eps, warmup_steps),
              "    steps = %d;" % steps, "    seed = %d;" % seed, "    device = cpu;", "}"]
    return "\n".join(lines) + "\n"


def default_masked_rows(rows, rate=0.15):
    """Capacity of the masked-row gather: expected selected rows plus 8 standard deviations, up to
    a multiple of 64, at most `rows` (832 for 4096 rows at 0.15)."""
    import math
    rate = min(1.0, max(0.0, rate))
    bound = rows * rate + 8.0 * math.sqrt(rows * rate * (1.0 - rate))
    return min(rows, (int(math.ceil(bound)) + 63) // 64 * 64)


# The benchmark configurations, by the short names the benchmark and the tests use.
CONFIGS = {
    "mlp": dict(kind="mlp", source=lambda **kw: mlp_classifier(**kw), rows=64),
    "encoder_block": dict(kind="block", source=lambda **kw: transformer_block(
        **{**dict(batch=32, layers=1, dropout=0.1, optimizer="adamw", lr=1e-3, weight_decay=0.01, eps=1e-6,
                  warmup_steps=0), **kw}), rows=4096),
    "bert_tiny": dict(kind="bert", source=lambda **kw: bert(**kw), rows=4096, seq=128, batch=32, vocab=30522),
    "bert_mini": dict(kind="bert", source=lambda **kw: bert(**{**dict(name="BertMini", layers=4, hidden=256, heads=4, ffn=1024), **kw}),
                      rows=4096, seq=128, batch=32, vocab=30522),
    "bert_base": dict(kind="bert", source=lambda **kw: bert(**{**dict(name="BertBase", layers=12, hidden=768, heads=12, ffn=3072,
                                                                      seq=512), **kw}),
                      rows=16384, seq=512, batch=32, vocab=30522),
}
