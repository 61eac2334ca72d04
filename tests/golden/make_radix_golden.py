"""Generates the radix-tree / prefix-cache golden fixtures.

    python tests/golden/make_radix_golden.py        (needs the reference checkout)

Writes seeded call scripts (radix_script_*.txt) and runs them through
oracle/_ref/radix_trace_ref -- oracle/radix_trace.cpp compiled against the REFERENCE's
radix_tree.h / prefix_cache.h (make -C oracle ref) -- to produce radix_expected_*.txt.
Both are committed; tests replay the scripts through this repository's own headers and
require identical text.  Scripts avoid what the reference leaves unspecified: eviction
candidates always have distinct timestamps ('tick' between the calls that stamp them).
"""
import random
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
REF_BIN = ROOT / "oracle" / "_ref" / "radix_trace_ref"


def toks(seq):
    return f"{len(seq)} " + " ".join(map(str, seq))


def script_tree(seed, n_ops, vocab):
    rnd = random.Random(seed)
    lines = [f"# tree script seed={seed}"]
    known = []
    for _ in range(n_ops):
        r = rnd.random()
        if known and rnd.random() < 0.6:
            base = rnd.choice(known)
            cut = rnd.randint(0, len(base))
            seq = base[:cut] + [rnd.randrange(vocab) for _ in range(rnd.randint(0, 6))]
        else:
            seq = [rnd.randrange(vocab) for _ in range(rnd.randint(0, 12))]
        if r < 0.35:
            ln = len(seq) if rnd.random() < 0.8 else len(seq) + rnd.randint(0, 3)
            lines.append("tick")
            lines.append(f"T insert {rnd.randint(0, 5)} {ln} {toks(seq)}")
            known.append(seq)
        elif r < 0.60:
            lines.append(f"T find {toks(seq)}")
        elif r < 0.68:
            lines.append(f"T contains {toks(seq)}")
        elif r < 0.74:
            lines.append(f"T remove {toks(seq)}")
        elif r < 0.82:
            lines.append("tick")
            lines.append(f"T addref {toks(seq)}")
        elif r < 0.88:
            lines.append(f"T release {toks(seq)}")
        elif r < 0.93:
            lines.append(f"T evict {rnd.randint(0, 60)}")
        elif r < 0.99:
            lines.append("T stats")
        else:
            lines.append("T clear")
            known = []
    lines.append("T stats")
    return lines


def script_cache(seed, n_req, vocab, capacity):
    rnd = random.Random(seed)
    lines = [f"# prefix-cache script seed={seed}",
             f"P config {capacity} {rnd.choice([1, 2, 4])} 1 0.9 1"]
    sessions = []
    held = []
    for i in range(n_req):
        if sessions and rnd.random() < 0.7:
            base = rnd.choice(sessions)
            seq = base[:rnd.randint(0, len(base))] + [rnd.randrange(vocab) for _ in range(rnd.randint(0, 20))]
        else:
            seq = [rnd.randrange(vocab) for _ in range(rnd.randint(0, 40))]
        lines.append(f"P match {toks(seq)}")
        held.append(seq)
        lines.append("tick")
        lines.append(f"P insert 0 {len(seq)} {toks(seq)}")
        sessions.append(seq)
        if held and rnd.random() < 0.5:
            h = held.pop(rnd.randrange(len(held)))
            # release by every prefix length: only the matched one changes a count, the
            # others must be no-ops or exact-length hits exactly as in the reference
            lines.append(f"P release {toks(h[:rnd.randint(0, len(h))])}")
        if rnd.random() < 0.1:
            lines.append(f"P remove {toks(rnd.choice(sessions))}")
        if rnd.random() < 0.15:
            lines.append("P stats")
            lines.append("P treestats")
            lines.append("P usage")
        if rnd.random() < 0.05:
            lines.append(f"P evict {rnd.randint(0, capacity)}")
    lines += ["P stats", "P treestats", "P cached"]
    return lines


def script_config4():
    """The shared-prefix token pattern at reduced count: common 1024-id prefix + unique
    256-id suffixes, ids uniform over [0,151936); the prefix itself is inserted so later
    requests hit it (a prefix shared only inside longer sequences is a miss)."""
    rnd = random.Random(4)
    prefix = [rnd.randrange(151936) for _ in range(1024)]
    lines = ["# config-4 pattern", "P config 65536 4 1 0.9 1"]
    for i in range(24):
        seq = prefix + [rnd.randrange(151936) for _ in range(256)]
        lines.append(f"P match {toks(seq)}")
        lines.append("tick")
        if i == 0:
            lines.append(f"P insert 0 1024 {toks(prefix)}")
        lines.append(f"P insert 0 {len(seq)} {toks(seq)}")
        lines.append(f"P release {toks(prefix)}")
        if i % 6 == 5:
            lines += ["P stats", "P treestats"]
    lines += ["P stats", "P treestats", "P cached", "P usage"]
    return lines


def main():
    if not REF_BIN.exists():
        subprocess.run(["make", "-C", str(ROOT / "oracle"), "ref"], check=True)
    jobs = {
        "tree_a": script_tree(11, 900, 6),
        "tree_b": script_tree(12, 900, 40),
        "cache_a": script_cache(21, 300, 12, 600),
        "cache_b": script_cache(22, 200, 50, 100000),
        "config4": script_config4(),
    }
    for name, lines in jobs.items():
        script = HERE / f"radix_script_{name}.txt"
        script.write_text("\n".join(lines) + "\n")
        out = subprocess.run([str(REF_BIN), str(script)], check=True, capture_output=True, text=True).stdout
        (HERE / f"radix_expected_{name}.txt").write_text(out)
        print(name, len(lines), "script lines,", out.count("\n"), "result lines")


if __name__ == "__main__":
    main()
