"""The reference's own benchmark drivers, unmodified, on top of this package's module mirror.

The drivers put their own directory first on sys.path and then ``from DSA import ...``
(sparse_attn/bench_sparse_attention_kernels.py:63-83, bench_sparse_attention_modules.py:73-85);
pre-seeding ``sys.modules["DSA"]`` with llmdivedeep_b200.DSA makes every name they import resolve
to the mirror.  Each driver runs in a child process from the unmodified copy under baseline/_ref
(staged by ``__graft_entry__.build()`` where a reference checkout is present; git-ignored) and
must print its tables without an error row."""
import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref", "sparse_attn")

SHIM = """
import runpy, sys
sys.path.insert(0, {root!r})
import llmdivedeep_b200.DSA as mirror
sys.modules["DSA"] = mirror
sys.argv = {argv!r}
runpy.run_path({script!r}, run_name="__main__")
"""


def _run_driver(script, args):
    path = os.path.join(REF, script)
    if not os.path.exists(path):
        pytest.skip("no reference copy under baseline/_ref (run __graft_entry__.build() next to a reference checkout)")
    code = SHIM.format(root=ROOT, argv=[script] + args, script=path)
    p = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert " err" not in p.stdout and "OOM" not in p.stdout and "MISSING" not in p.stdout, p.stdout
    return p.stdout


def _rows(out, seq_len, n_numbers):
    """Table rows that start with seq_len followed by at least n_numbers numeric fields."""
    rows = []
    for line in out.splitlines():
        f = line.split()
        if f and f[0] == str(seq_len) and len(f) > n_numbers:
            rows.append(f)
    return rows


def test_kernel_driver_runs_its_indexer_and_block_sparse_parts():
    out = _run_driver("bench_sparse_attention_kernels.py",
                      ["--indexer", "--sparse_gqa", "--seq_lens", "8192", "--warmup", "2", "--iters", "3"])
    assert "libdsa_b200" in out and "deep_gemm.fp8_mqa_logits: present" in out
    rows = _rows(out, 8192, 4)
    assert len(rows) >= 2, out                       # one PART B row, one PART C row
    # PART B row: seq_len sparsity sparse_ms dense_ms speedup TFLOPS (no dense backend here: nan in two columns);
    # PART C row: seq_len proj quant logits+topk total GB/s
    part_b = [r for r in rows if len(r) == 6 and "nan" in r]
    part_c = [r for r in rows if len(r) == 6 and "nan" not in r]
    assert part_b and float(part_b[0][2]) > 0 and float(part_b[0][5]) > 0, out
    assert part_c and all(float(v) > 0 for v in part_c[0][1:]), out
    print(out)


def test_module_driver_runs_all_three_indexer_modules():
    out = _run_driver("bench_sparse_attention_modules.py",
                      ["--all", "--seq_lens", "8192", "--warmup", "2", "--iters", "3"])
    assert out.count("indexer module") == 3
    rows = _rows(out, 8192, 8)
    assert len(rows) == 3, out
    for r in rows:
        proj, quant, logits, total = (float(v) for v in r[1:5])
        assert proj > 0 and quant > 0 and total > 0, r
    assert not re.search(r"Traceback", out)
    print(out)
