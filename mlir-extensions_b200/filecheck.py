"""A small FileCheck: enough of LLVM's tool for the reference's hot-path tests.

The reference pipes the runner's output into `FileCheck <test file>`
(tools/imex-runner/imex-runner.py.in:199-209).  Supported directives:
CHECK, CHECK-NEXT, CHECK-SAME, CHECK-NOT, CHECK-LABEL (as CHECK), with
`{{regex}}` blocks; horizontal whitespace is canonicalised on both sides, as
FileCheck does by default (the reference's tests rely on it: `[14.1,   14.8]`
and `[136, 136]` are checks against the same printer).
"""
import re
import sys


def _canon(s):
    return re.sub(r"[ \t]+", " ", s.strip())


def _pattern(text):
    out, pos = [], 0
    text = _canon(text)
    for m in re.finditer(r"\{\{(.*?)\}\}", text):
        out.append(re.escape(text[pos:m.start()]))
        out.append("(?:" + m.group(1) + ")")
        pos = m.end()
    out.append(re.escape(text[pos:]))
    return re.compile("".join(out))


def parse_checks(test_text, prefix="CHECK"):
    checks = []
    rx = re.compile(r"(?://|#|;)\s*" + re.escape(prefix) + r"(-NEXT|-SAME|-NOT|-LABEL|-DAG|-COUNT-\d+)?:\s?(.*)$")
    for line in test_text.splitlines():
        m = rx.search(line)
        if m:
            kind = (m.group(1) or "").lstrip("-") or "CHECK"
            checks.append((kind, m.group(2)))
    return checks


def check(output, test_text, prefix="CHECK"):
    """Returns None when every directive matches, else an error message."""
    checks = parse_checks(test_text, prefix)
    if not checks:
        return f"no {prefix} directives found"
    lines = [_canon(l) for l in output.splitlines()]
    li, col = 0, 0       # search position: line index and column in that line
    last_line = -1       # line of the last positive match
    pending_not = []
    for kind, text in checks:
        pat = _pattern(text)
        if kind == "NOT":
            pending_not.append((pat, text))
            continue
        reps = 1
        if kind.startswith("COUNT-"):
            reps = int(kind.split("-")[1])
            kind = "CHECK"
        for _ in range(reps):
            found = None
            if kind == "SAME":
                if last_line < 0:
                    return f"{prefix}-SAME without a previous match: {text}"
                m = pat.search(lines[last_line], col)
                if m:
                    found = (last_line, m.end())
            elif kind == "NEXT":
                if last_line < 0:
                    return f"{prefix}-NEXT without a previous match: {text}"
                nxt = last_line + 1
                if nxt < len(lines):
                    m = pat.search(lines[nxt])
                    if m:
                        found = (nxt, m.end())
            else:  # CHECK / LABEL / DAG (DAG treated as ordered)
                start_col = col
                for i in range(li, len(lines)):
                    m = pat.search(lines[i], start_col if i == li else 0)
                    if m:
                        found = (i, m.end())
                        break
            if not found:
                ctx = "\n".join(lines[max(0, last_line):last_line + 4])
                return f"{prefix}{'' if kind == 'CHECK' else '-' + kind}: expected string not found: {text}\nnear:\n{ctx}"
            for npat, ntext in pending_not:
                for i in range(max(last_line, 0), found[0] + 1):
                    if npat.search(lines[i]):
                        return f"{prefix}-NOT: excluded string found: {ntext}"
            pending_not = []
            last_line, col = found
            li = last_line
    for npat, ntext in pending_not:
        for i in range(max(last_line, 0), len(lines)):
            if npat.search(lines[i]):
                return f"{prefix}-NOT: excluded string found: {ntext}"
    return None


def main(argv=None):
    import argparse
    ap = argparse.ArgumentParser(description="FileCheck-style checker (reads the output on stdin)")
    ap.add_argument("check_file")
    ap.add_argument("--check-prefix", default="CHECK")
    a = ap.parse_args(argv)
    err = check(sys.stdin.read(), open(a.check_file).read(), a.check_prefix)
    if err:
        print(f"{a.check_file}: error: {err}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    sys.exit(main())
