#!/usr/bin/env python3
"""bench_imex for the B200 runtime — the reference's benchmark driver, same report.

The reference builds its benchmark grid at configure time (each
benchmarks/<name>/CMakeLists.txt fills <name>_gpu.mlir.in from <name>.shapes.in
and <name>.dtypes.in) and benchmarks/bench_imex.in then runs every generated
.mlir through imex-runner with IMEX_ENABLE_PROFILING=1, keeping the lines that
hold "execution time" in report.txt.  This script does both steps:

    bench_imex.py -b --benchmarks <reference>/benchmarks [relu | softmax | ... | file.mlir | folder]

    -b   run on the B200 runtime (where the reference has -l / -s for its two runtimes)
    -c   the reference's CPU run: refused, this build has no CPU execution path

With --emit-plan nothing is launched: the report lists the kernels each
benchmark becomes (works on a machine without a GPU).
"""
import argparse
import datetime
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
IMEX_RUNNER = os.path.join(HERE, "imex_runner.py")

BENCHMARKS = ["relu", "silu", "softmax", "transpose", "reduce", "kLoopFusion", "kInputFusion"]


def _lines(path):
    with open(path) as f:
        return [l.strip() for l in f if l.strip()]


def _fill(template, out_path, subst):
    text = open(template).read()
    for key, value in subst.items():
        text = text.replace("@" + key + "@", value)
    os.makedirs(os.path.dirname(out_path), exist_ok=True)
    with open(out_path, "w") as f:
        f.write(text)
    return out_path


def instantiate(bench_root, name, out_root):
    """The .mlir files the reference's CMake generates for benchmark `name`
    (gpu flavour), written under out_root/<name>/gpu/; returns their paths."""
    src = os.path.join(bench_root, name)
    dtypes = _lines(os.path.join(src, name + ".dtypes.in"))
    out = []
    if name in ("relu", "silu"):  # benchmarks/relu/CMakeLists.txt:4-28
        for shape in _lines(os.path.join(src, name + ".shapes.in")):
            rank = shape.count("x") + 1
            subst = {"shape": shape, "affine_map": ", ".join("d%d" % i for i in range(rank)),
                     "iterator_types": ", ".join(['"parallel"'] * rank)}
            for dt in dtypes:
                out.append(_fill(os.path.join(src, name + "_gpu.mlir.in"),
                                 os.path.join(out_root, name, "gpu", "%s_%s_%s.mlir" % (name, shape, dt)),
                                 dict(subst, dtype=dt)))
    elif name == "softmax":  # benchmarks/softmax/CMakeLists.txt:4-21
        for shape in _lines(os.path.join(src, "softmax.shapes.in")):
            sizes = shape.split("x")
            if len(sizes) > 2:
                print("Unsupported shape for softmax: " + shape, file=sys.stderr)
                continue
            for dt in dtypes:
                out.append(_fill(os.path.join(src, "softmax_gpu.mlir.in"),
                                 os.path.join(out_root, name, "gpu", "softmax_%s_%s.mlir" % (shape, dt)),
                                 {"shape": shape, "batch_size": sizes[0], "dtype": dt}))
    elif name == "transpose":  # benchmarks/transpose/CMakeLists.txt:4-25
        for in_shape in _lines(os.path.join(src, "transpose.shapes.in")):
            sizes = in_shape.split("x")
            if len(sizes) not in (2, 3):
                print("Unsupported shape for transpose " + in_shape, file=sys.stderr)
                continue
            template = "transpose%dd_gpu.mlir.in" % len(sizes)
            for dt in dtypes:
                out.append(_fill(os.path.join(src, template),
                                 os.path.join(out_root, name, "gpu", "transpose_%s_%s.mlir" % (in_shape, dt)),
                                 {"in_shape": in_shape, "out_shape": "x".join(reversed(sizes)), "dtype": dt}))
    elif name == "reduce":  # benchmarks/reduce/CMakeLists.txt:1-9 (the shape is in the file name only)
        for dt in dtypes:
            out.append(_fill(os.path.join(src, "reduce_gpu.mlir.in"),
                             os.path.join(out_root, name, "gpu", "reduce_1x16x512x512_%s.mlir" % dt),
                             {"dtype": dt}))
    elif name in ("kLoopFusion", "kInputFusion"):  # benchmarks/kLoopFusion/CMakeLists.txt:1-8
        for dt in dtypes:
            out.append(_fill(os.path.join(src, name + ".mlir.in"),
                             os.path.join(out_root, name, "%s_512x1024_%s.mlir" % (name, dt)),
                             {"dtype": dt}))
    else:
        raise ValueError("unknown benchmark " + name)
    return out


def find_tests(target, bench_root, out_root):
    if target is None:
        return [p for b in BENCHMARKS for p in instantiate(bench_root, b, out_root)]
    if target in BENCHMARKS:
        return instantiate(bench_root, target, out_root)
    if os.path.isdir(target):
        found = []
        for d, _, files in os.walk(target):
            found += [os.path.join(d, f) for f in files if f.endswith(".mlir")]
        return sorted(found)
    if os.path.isfile(target):
        if not target.endswith(".mlir"):
            sys.exit("Only take .mlir file")
        return [target]
    sys.exit("no such benchmark, folder or file: " + target)


def run_one(path, pipeline, emit_plan):
    cmd = [sys.executable, IMEX_RUNNER, "-i", path, "-e", "main", "--entry-point-result=void"]
    if pipeline:
        cmd += ["--pass-pipeline-file=" + pipeline]
    if emit_plan:
        cmd.append("--emit-plan")
    env = dict(os.environ, IMEX_ENABLE_PROFILING="1")
    r = subprocess.run(cmd, capture_output=True, text=True, env=env)
    return r.returncode, r.stdout, r.stderr


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("-b", action="store_true", dest="b200", help="run on the B200 runtime")
    ap.add_argument("-c", action="store_true", dest="cpu", help="the reference's CPU run (refused here)")
    ap.add_argument("--benchmarks", default=None, help="the reference's benchmarks/ folder (templates)")
    ap.add_argument("--out", default="imex_benchmarks", help="where the instantiated .mlir files go")
    ap.add_argument("--report", default="report.txt")
    ap.add_argument("--emit-plan", action="store_true", help="list the kernels instead of running them")
    ap.add_argument("target", nargs="?", default=None,
                    help="a benchmark name, a folder containing .mlir files or an .mlir file")
    args = ap.parse_args(argv)
    if args.cpu:
        sys.exit("Running on CPU is not available: this build has no CPU execution path (use -b)")
    if not args.b200:
        sys.exit("Please select a runtime. using '%s -h' for more usage info" % os.path.basename(sys.argv[0]))
    needs_templates = args.target is None or args.target in BENCHMARKS
    if needs_templates and not args.benchmarks:
        sys.exit("--benchmarks <reference>/benchmarks is needed to instantiate the benchmark templates")
    print("Running on GPU using the B200 runtime")
    tests = find_tests(args.target, args.benchmarks, args.out)
    print("Run the following Tests:")
    print("\n".join(tests) + "\n")
    pipeline = None
    if args.benchmarks and os.path.exists(os.path.join(args.benchmarks, "pipelines", "linalg-to-gpu.pp")):
        pipeline = os.path.join(args.benchmarks, "pipelines", "linalg-to-gpu.pp")
    failed = 0
    with open(args.report, "w") as report:
        report.write("\n================ Imex Perf (B200) @ %s ================\n\n"
                     % datetime.datetime.now().strftime("%c"))
        for path in tests:
            name = os.path.basename(path)
            rc, out, err = run_one(path, pipeline, args.emit_plan)
            print("%s: %s" % (name, " ".join(out.split()) if rc == 0 else "FAILED: " + err.strip().splitlines()[-1]
                                if err.strip() else "FAILED"))
            if rc != 0:
                failed += 1
                report.write("%s: FAILED (%s)\n" % (name, err.strip().splitlines()[-1] if err.strip() else rc))
                continue
            wanted = "kernel " if args.emit_plan else "execution time"
            for line in out.splitlines():
                if wanted in line:
                    report.write("%s: %s\n" % (name, line))
    return 1 if failed else 0


if __name__ == "__main__":
    sys.exit(main())
