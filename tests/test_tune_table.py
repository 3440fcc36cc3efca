"""The planner's tuning table (written by abq-llm_b200/tune.py, the timed search that replaces the reference's list of tile
instantiations): a line for a problem changes its launch shape, problems without a line keep the heuristic, a `planes` entry
sends a prepared-weights request to the kernel that reads the planes.  Planning only: no GPU needed."""
import os
import subprocess
import sys
import textwrap
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

PLAN = textwrap.dedent("""
    import sys, ctypes
    sys.path.insert(0, {tests!r}); sys.path.insert(0, {root!r})
    from conftest import load_package
    abq = load_package()
    from abq_llm_b200 import binding as B
    for (M, N, K) in ((4, 2048, 1024), (4, 4096, 1024)):
        p = B.GemmParams(); p.M, p.N, p.K = M, N, K; p.X = p.W = p.D = 4096; p.x_bits, p.w_bits, p.x_signed = 8, 4, 1
        p.route = 2; p.flags = abq.FLAG_WEIGHTS_PREPARED; p.w_prepared = 4096
        st = B.GemmState(); rc = abq.lib().abq_gemm_init(ctypes.byref(p), ctypes.byref(st))
        print(st.grid[0], st.block[0], st.tile[3], rc)
""")


def plan(env):
    code = PLAN.format(tests=str(ROOT / "tests"), root=str(ROOT))
    e = {k: v for k, v in os.environ.items() if not k.startswith("ABQ_")}
    e.update(env)
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=e, timeout=300)
    assert out.returncode == 0, out.stderr[-1500:]
    return [tuple(int(v) for v in line.split()) for line in out.stdout.strip().splitlines()]


def test_table_entry_changes_the_plan(tmp_path):
    table = tmp_path / "t.txt"
    table.write_text("# comment\n4 8 4 2048 1024 0 0 : 0 0 0 16 1 74 0 0 0   # sixteen warps, one CTA per SM, 74 CTAs\n")
    base = plan({"ABQ_TUNE_IGNORE": "1"})
    tuned = plan({"ABQ_TUNE_TABLE": str(table)})
    assert tuned[0][:2] == (74, 512) and base[0][:2] != (74, 512) and tuned[0][3] == 0
    assert tuned[1] == base[1]                      # no line for the second problem: heuristic
    assert plan({"ABQ_TUNE_TABLE": str(table), "ABQ_TUNE_IGNORE": "1"}) == base
    assert plan({"ABQ_TUNE_TABLE": str(table), "ABQ_STREAM_CTAS": "37"})[0][0] == 37   # the environment outranks the table


def test_planes_entry_falls_back_to_the_plane_kernel(tmp_path):
    table = tmp_path / "t.txt"
    table.write_text("4 8 4 2048 1024 0 0 : 0 0 0 0 0 0 0 0 1\n")
    tuned = plan({"ABQ_TUNE_TABLE": str(table)})
    base = plan({"ABQ_TUNE_IGNORE": "1"})
    # the plane kernel's plan needs a TMA descriptor from the driver: on a box without one the call answers ABQ_ERR_CUDA (4),
    # which also shows that the prepared-weights plan was not taken; with a driver it is the plane kernel's 16-warp CTA
    assert tuned[0][3] == 4 or (tuned[0][3] == 0 and tuned[0][1] == 512)
    assert tuned[0] != base[0] and base[0][3] == 0
    assert tuned[1] == base[1]


def test_committed_table_parses():
    table = ROOT / "abq-llm_b200" / "abq_tune_table.txt"
    if not table.exists():
        return
    for line in table.read_text().splitlines():
        if not line.strip() or line.startswith("#"):
            continue
        key, _, rest = line.partition(":")
        assert len(key.split()) == 7 and len(rest.split("#")[0].split()) == 9, line


INVARIANTS = textwrap.dedent("""
    import sys, ctypes
    sys.path.insert(0, {tests!r}); sys.path.insert(0, {root!r})
    from conftest import load_package
    abq = load_package()
    from abq_llm_b200 import binding as B
    bad = []
    n = 0
    for q in (2, 3, 4, 8):
        for M in (1, 2, 3, 4, 7, 8):                       # (9 and more token rows may need a K split: its counters are device memory)
            for (N, K) in ((16, 128), (48, 384), (4096, 4096), (12288, 4096), (11008, 4096), (4096, 11008), (5120, 5120), (13824, 5120), (1000, 1152)):
                for group in (0, 64, 128):
                    if group and K % group:
                        continue
                    p = B.GemmParams(); p.M, p.N, p.K = M, N, K; p.X = p.W = p.D = 4096; p.x_bits, p.w_bits, p.x_signed = 8, q, 1
                    p.route = 2; p.flags = abq.FLAG_WEIGHTS_PREPARED; p.w_prepared = 4096
                    if group:
                        p.out_dtype, p.scale_mode, p.group_size, p.w_scale = 1, abq.SCALE_GROUP, group, 4096
                    st = B.GemmState(); rc = abq.lib().abq_gemm_init(ctypes.byref(p), ctypes.byref(st))
                    n += 1
                    if rc == 4 and st.cluster == 0:
                        continue                            # a shape that splits K: planned, but the counter reset needs a device
                    ok = (rc == 0 and abq.state_kernel(st) == "stream_kernel" and st.block[0] in (64, 128, 256, 512) and 1 <= st.grid[0] <= 2048
                          and st.shared_mem_size <= 227 * 1024 and st.tile[1] >= 2 and st.tile[3] >= 1)
                    if not ok:
                        bad.append((q, M, N, K, group, rc, st.grid[0], st.block[0], st.shared_mem_size, list(st.tile)))
    print(n, bad)
""")


def test_prepared_weights_plans_stay_inside_the_hardware_limits():
    """Every decode problem of up to 8 tokens over a spread of shapes, widths and scale groups gets a prepared-weights plan:
    a power-of-two CTA of at most 16 warps, at most 227 KB of shared memory, a ring of at least two chunks per warp."""
    code = INVARIANTS.format(tests=str(ROOT / "tests"), root=str(ROOT))
    e = {k: v for k, v in os.environ.items() if not k.startswith("ABQ_")}
    e["ABQ_TUNE_IGNORE"] = "1"
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=e, timeout=600)
    assert out.returncode == 0, out.stderr[-1500:]
    count, bad = out.stdout.strip().split(" ", 1)
    assert int(count) > 500 and bad == "[]", bad[:2000]
