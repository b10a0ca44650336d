"""`python -m modelspec_b200 train|infer <file.mspec>`: the reference's `modelspec train|infer
--backend cuda` on this backend, printing the reference's standard output for the run
(crates/modelspec-cli/src/train.rs:7-17; crates/modelspec-cli/src/infer.rs:1-60).

    python -m modelspec_b200 train FILE [--data DIR] [--eval DIR] [--eval-every N] [--masked-rows N]
        [--resume IN.msckpt] [--checkpoint OUT.msckpt] [--stats] [--profile] [--bf16] [--device I]
    python -m modelspec_b200 infer FILE [--resume IN.msckpt] [--bf16] [--device I]

`--data DIR` is a packed masked-language-model directory when it holds `binding.json`, else a dense
one (`<name>.f32` / `<name>.i32` per declaration, optional `order.u32`; train/data.rs:1443-1483).
Without `--data` the run trains on the reference's synthetic batch (one f32 input, one f32 target).
Diagnostics go to standard error and the exit status is 1, as the reference's CLI answers.
"""
import argparse
import os
import sys

import modelspec_b200 as M


def infer_function(args):
    """`infer <file> --resume <ckpt> --data <dir> --function <name> --out <path>`
    (crates/modelspec-cli/src/infer.rs:306-470): one line,
    `function <name> blocks <blocks> rows <rows> out <path>`."""
    run = device = None
    try:
        source = open(args.file).read()
        device = M.Device(args.device)
        run = M.Training(device, source, 0, M.PLAN_BF16 if args.bf16 else M.PLAN_DEFAULT, function=args.function)
        run.refuse_out_reading(args.data, args.out, args.file, args.resume)
        if args.resume:
            loaded = M.Checkpoint.read(args.resume)
            try:
                run.load_parameters(loaded)
            finally:
                loaded.destroy()
        blocks, rows = run.infer_dense(args.data, args.out)
        sys.stdout.write("function %s blocks %d rows %d out %s\n" % (args.function, blocks, rows, args.out))
        return 0
    except (M.MsxError, OSError) as error:
        sys.stderr.write("error: %s\n" % error)
        return 1
    finally:
        if run is not None:
            run.destroy()
        if device is not None:
            device.close()


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m modelspec_b200")
    ap.add_argument("command", choices=["train", "infer"])
    ap.add_argument("file")
    ap.add_argument("--data", help="a packed masked-language-model directory (it holds binding.json) or a dense one")
    ap.add_argument("--eval", help="a dense directory to evaluate the trained parameters on (a last line `eval loss=... accuracy=...`)")
    ap.add_argument("--eval-every", type=int, default=0, help="evaluate the HeldOut split of --data every N steps and at the last step")
    ap.add_argument("--masked-rows", type=int, default=0, help="capacity of the masked-row gather (0: none)")
    ap.add_argument("--resume", help="a .msckpt checkpoint to start from")
    ap.add_argument("--checkpoint", help="write the state after the last step here")
    ap.add_argument("--stats", action="store_true")
    ap.add_argument("--profile", action="store_true")
    ap.add_argument("--bf16", action="store_true", help="a mixed-precision plan (bf16 storage and products, f32 masters)")
    ap.add_argument("--function", help="infer: run this model function over the dense directory --data (with --out)")
    ap.add_argument("--out", help="infer --function: the file the function's results go to, one row per sample, f32")
    ap.add_argument("--device", type=int, default=0)
    args = ap.parse_args(argv)
    if args.command == "infer" and (args.function or args.out):
        # `--function` or `--out` without `--data`, and `--data` without both, is a usage error.
        if not (args.data and args.function and args.out):
            ap.error("infer --function needs --data, --function and --out together")
        return infer_function(args)
    packed = run = device = None
    try:
        source = open(args.file).read()
        device = M.Device(args.device)
        run = M.Training(device, source, args.masked_rows, M.PLAN_BF16 if args.bf16 else M.PLAN_DEFAULT)
        if args.data and os.path.exists(os.path.join(args.data, "binding.json")):
            packed = M.Packed(args.data)
            run.bind_packed(packed)
            if args.eval_every > 0:
                run.heldout_packed()
            run.feed_packed(0)
        elif args.data:
            run.bind_dense(args.data)
            run.feed_dense(0)
        else:
            run.synthetic()
        start = 0
        if args.resume:
            loaded = M.Checkpoint.read(args.resume)
            start = run.resume(loaded)
            loaded.destroy()
        if args.command == "infer":
            sys.stdout.write(run.infer_report())
            return 0
        try:
            sys.stdout.write(run.run(start, args.eval_every))
        except M.MsxError:
            sys.stdout.write(run.report())  # the lines through the failing step
            raise
        if args.eval:
            sys.stdout.write(M.eval_line(*run.eval_dense(args.eval)))
        if args.checkpoint:
            done = run.checkpoint(start + run.steps)
            done.write(args.checkpoint)
            done.destroy()
        if args.stats:
            sys.stdout.write(run.step_plan.stats_report())
        if args.profile:
            sys.stdout.write(run.step_plan.profile_report(run.forward_plan))
        return 0
    except (M.MsxError, OSError) as error:
        sys.stderr.write("error: %s\n" % error)
        return 1
    finally:
        if run is not None:
            run.destroy()
        if packed is not None:
            packed.close()
        if device is not None:
            device.close()


if __name__ == "__main__":
    sys.exit(main())
