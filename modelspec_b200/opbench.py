"""Times one kernel of the backend on its own, through the C ABI, on device buffers of the
caller's: the entry points `msx_op_matmul`, `msx_op_matmul_bf16` and `msx_op_attention_bf16` exist
for exactly this (a single kernel on a small case, for `ncu` and for tuning).

    python -m modelspec_b200.opbench matmul_bf16 M N K [--form nn|nt|tn|tt] [--f32-out] [--reps R]
    python -m modelspec_b200.opbench matmul_f32 M N K [--form ...] [--exact] [--reps R]
    python -m modelspec_b200.opbench attention_bf16 BATCH SEQ HEADS HEAD_DIM [--forward-only] [--reps R]
    python -m modelspec_b200.opbench heldout_rows ROWS CLASSES [--selected FRACTION] [--reps R]

Prints one line: milliseconds per call (CUDA events on the launching stream, after 3 warm-up
calls) and the algorithmic rate (2 m n k FLOP for a product; 4 b a s^2 d forward and 10 b a s^2 d
backward for attention; one read of the logits, 4 rows classes bytes, for the held-out reduction,
whose result is also checked against a float64 restatement in torch). torch only provides the device buffers, the stream and the events.
"""
import argparse
import ctypes as C
import sys

import modelspec_b200 as M


def timed(torch, go, reps):
    for _ in range(3):
        go()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(reps):
        go()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / reps


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("op", choices=["matmul_bf16", "matmul_f32", "attention_bf16", "heldout_rows"])
    ap.add_argument("dims", type=int, nargs="+")
    ap.add_argument("--form", default="nn", choices=["nn", "nt", "tn", "tt"])
    ap.add_argument("--f32-out", action="store_true")
    ap.add_argument("--exact", action="store_true", help="matmul_f32: the exact fused-chain kernel instead of the tensor cores")
    ap.add_argument("--forward-only", action="store_true")
    ap.add_argument("--selected", type=float, default=0.15, help="fraction of rows of weight 1 (the rest have weight 0)")
    ap.add_argument("--reps", type=int, default=20)
    args = ap.parse_args()
    import torch

    L = M.lib()
    ptr = lambda t: C.c_void_p(t.data_ptr())
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    if args.op.startswith("matmul"):
        m, n, k = args.dims
        a_t, b_t = args.form[0] == "t", args.form[1] == "t"
        half = args.op == "matmul_bf16"
        dtype = torch.bfloat16 if half else torch.float32
        a = torch.randn((k, m) if a_t else (m, k), device="cuda").to(dtype)
        b = torch.randn((n, k) if b_t else (k, n), device="cuda").to(dtype)
        c = torch.empty((m, n), dtype=torch.float32 if (args.f32_out or not half) else torch.bfloat16, device="cuda")
        need = (L.msx_op_matmul_bf16_workspace if half else L.msx_op_matmul_workspace)(m, n, k)
        ws = torch.empty(max(need, 1), dtype=torch.float32, device="cuda")

        def go():
            if half:
                rc = L.msx_op_matmul_bf16(ptr(a), int(a_t), ptr(b), int(b_t), ptr(c), int(c.dtype == torch.bfloat16), m, n, k, ptr(ws), need,
                                          ptr(status), stream)
            else:
                rc = L.msx_op_matmul(ptr(a), int(a_t), ptr(b), int(b_t), ptr(c), m, n, k, ptr(ws), need, ptr(status), stream, int(args.exact))
            if rc != M.OK:
                raise SystemExit(L.msx_last_error(None).decode())

        ms = timed(torch, go, args.reps)
        print("%s %s m %d n %d k %d: %.4f ms, %.1f TFLOP/s, status %d" % (args.op, args.form, m, n, k, ms, 2.0 * m * n * k / ms / 1e9,
                                                                        int(status.item())))
        return
    if args.op == "heldout_rows":
        rows, classes = args.dims
        gen = torch.Generator(device="cuda").manual_seed(7)
        logits = torch.randn((rows, classes), device="cuda", generator=gen) * 3.0
        labels = torch.randint(0, classes, (rows,), device="cuda", generator=gen, dtype=torch.int32)
        weights = (torch.rand(rows, device="cuda", generator=gen) < args.selected).float()
        scratch = torch.empty(12 * rows, dtype=torch.uint8, device="cuda")
        state = torch.zeros(3, dtype=torch.int64, device="cuda")

        def go():
            state.zero_()
            rc = L.msx_op_heldout_rows(ptr(logits), 0, ptr(labels), ptr(weights), rows, classes, ptr(scratch), ptr(state), stream)
            if rc != M.OK:
                raise SystemExit(L.msx_last_error(None).decode())

        ms = timed(torch, go, args.reps)
        numerator = float(state[:1].view(torch.float64).item())
        correct = int(state[1].item())
        wide = logits.double()
        nll = torch.logsumexp(wide, 1) - wide.gather(1, labels.long()[:, None])[:, 0]
        expect = float((weights.double() * nll).sum().item())
        hits = int(((wide.argmax(1) == labels.long()) & (weights > 0)).sum().item())
        print("heldout_rows rows %d classes %d selected %.2f: %.4f ms, %.1f GB/s of one read; numerator %.9g (float64 %.9g), correct %d (%d)" % (
            rows, classes, args.selected, ms, 4.0 * rows * classes / ms / 1e6, numerator, expect, correct, hits))
        return
    batch, seq, heads, d = args.dims
    rows, h = batch * seq, heads * d
    q, k, v, g = (torch.randn((rows, h), device="cuda").to(torch.bfloat16) for _ in range(4))
    mask = torch.ones((batch, seq), dtype=torch.float32, device="cuda")
    out, dq, dk, dv = (torch.empty((rows, h), dtype=torch.bfloat16, device="cuda") for _ in range(4))
    stats = torch.empty(rows * heads * 2, dtype=torch.float32, device="cuda")

    def go():
        rc = L.msx_op_attention_bf16(ptr(q), ptr(k), ptr(v), ptr(mask), None if args.forward_only else ptr(g), ptr(out), ptr(dq), ptr(dk), ptr(dv),
                                     ptr(stats), batch, seq, seq, heads, d, ptr(status), stream)
        if rc != M.OK:
            raise SystemExit(L.msx_last_error(None).decode())

    ms = timed(torch, go, args.reps)
    flop = (4.0 if args.forward_only else 14.0) * batch * heads * seq * seq * d
    print("attention_bf16 %s batch %d seq %d heads %d d %d: %.4f ms, %.1f TFLOP/s, status %d" % (
        "forward" if args.forward_only else "forward + backward", batch, seq, heads, d, ms, flop / ms / 1e9, int(status.item())))


if __name__ == "__main__":
    sys.exit(main())
