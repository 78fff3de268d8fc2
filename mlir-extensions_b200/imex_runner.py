#!/usr/bin/env python3
"""imex-runner for the B200 path — same command line as the reference's driver.

The reference's imex-runner.py (tools/imex-runner/imex-runner.py.in:82-216)
runs `imex-opt --pass-pipeline=... | mlir-runner ... | FileCheck`.  This one
keeps its options (-i, -o, -f/--pass-pipeline-file, -p, -b, -a, -n, --filecheck,
--check-prefix, -d, -r/--runner, --requires, --igpu-fp64; unknown options go to
the runner) and runs `imex-b200-runner` instead of the imex-opt | mlir-runner
pair: the recogniser stands where the pass pipeline stood, so the pipeline text
is read (same flattening rules, lines joined with ',', '//' comments dropped)
but only reported with -d; it never becomes a literal pass list.  Every
pipeline — the reference's CPU one included — executes on the B200 runtime:
this build has no CPU execution path.  `--requires` lists features a RUN line
needs; the only runtime feature enabled here is `b200-runtime`, so the
reference's `l0-runtime` / `sycl-runtime` RUN lines exit 0 untouched, exactly
as they do in the reference when that runtime was not built
(imex-runner.py.in:113-115).
"""
import argparse
import os
import re
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
RUNNER = os.path.join(HERE, "bin", "imex-b200-runner")

ALL_FEATURES = ["vulkan-runner", "l0-runtime", "sycl-runtime", "igpu-fp64", "spirv-backend",
                "mlir-sycl-runtime", "mlir-levelzero-runtime", "b200-runtime"]
ENABLED_FEATURES = ["b200-runtime"]


def flatten_pipeline(path):
    """The reference's .pp flattening (imex-runner.py.in:117-136)."""
    pipeline = None
    with open(path) as f:
        for line in f:
            line = re.sub("//.*?\n", "", line).strip()
            if line:
                pipeline = ",".join([pipeline, line]) if pipeline else line
    if pipeline is None:
        return ""
    pipeline = re.sub(r",+", ",", pipeline.strip())
    pipeline = re.sub(r"\(,", "(", pipeline)
    pipeline = re.sub(r",\)", ")", pipeline)
    return pipeline.rstrip(",")


def main(argv=None):
    ap = argparse.ArgumentParser(description="run a func/linalg MLIR file on the B200 runtime, "
                                             "optionally piping the output into a FileCheck-style checker")
    ap.add_argument("--input-file", "-i", default=None)
    ap.add_argument("--output-file", "-o", default=None)
    ap.add_argument("--pass-pipeline-file", "-f", default=None)
    ap.add_argument("--pass-pipeline", "-p", default=None)
    ap.add_argument("--imex-print-before-all", "-b", action="store_true", dest="before")
    ap.add_argument("--imex-print-after-all", "-a", action="store_true", dest="after")
    ap.add_argument("--no-mlir-runner", "-n", action="store_true", dest="no_mlir_runner")
    ap.add_argument("--filecheck", action="store_true", dest="run_filecheck")
    ap.add_argument("--check-prefix", default=None)
    ap.add_argument("--debug", "-d", action="store_true")
    ap.add_argument("--runner", "-r", default="mlir-runner", choices=["mlir-runner", "imex-b200-runner"])
    ap.add_argument("--requires", default=",".join(ENABLED_FEATURES))
    ap.add_argument("--igpu-fp64", action="store_true", dest="igpu_has_fp64")
    ap.add_argument("--no-igpu-fp64", action="store_false", dest="igpu_has_fp64")
    args, unknown = ap.parse_known_args(argv)

    required = [r for r in args.requires.split(",") if r]
    if not set(required) <= set(ALL_FEATURES):
        print("Invalid option passed to --requires")
        print("your options were: ", *required)
        print("valid options are: ", *ALL_FEATURES)
        return 1
    if not set(required) <= set(ENABLED_FEATURES):
        return 0  # feature not built: the RUN line is skipped, as in the reference
    if not args.input_file:
        print("Error: --input-file is required")
        return 1
    if not os.path.exists(RUNNER):
        print(f"Error: {RUNNER} is missing: run `python mlir-extensions_b200/build.py`", file=sys.stderr)
        return 1
    pipeline = flatten_pipeline(args.pass_pipeline_file) if args.pass_pipeline_file else args.pass_pipeline
    if args.debug and pipeline:
        print(f"// pipeline (selects nothing here: every pipeline runs on the B200 runtime): {pipeline}",
              file=sys.stderr)

    cmd = [RUNNER, args.input_file]
    if args.no_mlir_runner:
        cmd.append("--emit-plan")  # nothing is executed: print the recognised kernels and ABI calls
    if args.before or args.after:
        cmd.append("--trace")
    cmd += unknown
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, text=True)
    if args.output_file:
        with open(args.output_file, "w") as f:
            f.write(proc.stdout)
    if args.run_filecheck and proc.returncode == 0:
        sys.path.insert(0, HERE)
        import filecheck
        err = filecheck.check(proc.stdout, open(args.input_file).read(), args.check_prefix or "CHECK")
        if err:
            sys.stdout.write(proc.stdout)
            print(f"{args.input_file}: error: {err}", file=sys.stderr)
            return 1
        return 0
    if not args.output_file:
        sys.stdout.write(proc.stdout)
    return proc.returncode


if __name__ == "__main__":
    sys.exit(main())
