"""Helpers to run a function as N gloo ranks in child processes."""
import os
import subprocess
import sys
import tempfile
import textwrap

from chatlearn_b200.utils.utils import get_free_port

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def run_ranks(script: str, nproc: int, timeout: int = 600, env=None, expect_fail=False):
    """Run ``script`` (python source) as ``nproc`` ranks; returns list of stdout."""
    port = get_free_port()
    with tempfile.NamedTemporaryFile("w", suffix=".py", delete=False) as f:
        f.write("import sys; sys.path.insert(0, %r)\n" % ROOT + textwrap.dedent(script))
        path = f.name
    procs = []
    for r in range(nproc):
        e = dict(os.environ)
        e.update(env or {})
        e.update(RANK=str(r), LOCAL_RANK=str(r), WORLD_SIZE=str(nproc), MASTER_ADDR="127.0.0.1",
                 MASTER_PORT=str(port), CHATLEARN_FORCE_CPU="1", OMP_NUM_THREADS="2")
        procs.append(subprocess.Popen([sys.executable, path], env=e, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs, codes = [], []
    for p in procs:
        try:
            out, _ = p.communicate(timeout=timeout)
        except subprocess.TimeoutExpired:
            p.kill()
            out, _ = p.communicate()
            out += "\n<<timeout>>"
        outs.append(out)
        codes.append(p.returncode)
    os.unlink(path)
    if not expect_fail:
        assert all(c == 0 for c in codes), "\n".join(f"--- rank {i} (rc={c}) ---\n{o[-3000:]}"
                                                      for i, (o, c) in enumerate(zip(outs, codes)))
    return outs, codes
