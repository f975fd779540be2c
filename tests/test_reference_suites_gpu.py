"""The reference project's own GPU test files, run unmodified against this backend.

`newt_b200.install_aliases()` makes `import newt` / `import deuteron` resolve here, so the
files of the reference's tests/ directory can be collected as they are.  They are not part of
this repository: point NEWT_REFERENCE_DIR at a checkout of the reference (the directory that
holds its tests/ folder) to run them; without it every case here is skipped.

Each file runs in a child process (its own CUDA context and module table).  A file passes
when every failing test in it is one of the cases listed in KNOWN below, each with the reason
this backend answers differently; anything else failing is a bug here.
"""

import os
import re
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

FILES = ["test_vector_add.py", "test_softmax_layernorm.py", "test_matmul.py", "test_deuteron.py",
         "test_ops.py", "test_control_flow.py", "test_review_fixes.py", "test_pipeline_dot.py",
         "test_runtime_smoke.py"]

# test id (as pytest prints it, without the file) -> why the result differs by design
KNOWN = {
    "test_review_fixes.py": {
        "test_pointer_rebase_rejected":
            "the reference refuses a loop-carried pointer that moves to another tensor (its loops "
            "keep one base per pointer, newt/compiler/codegen.py:826-865); here the pointer is an "
            "ordinary loop-carried value and the program runs (tests/generic_programs.py "
            "`switch_source` checks the result)",
        "test_int_storage_float_update_rejected":
            "a loop over a constexpr range is unrolled while tracing, so `s = 0; s = s + 0.5` is "
            "Python arithmetic on a Python number and yields 0.5 * ITERS; the reference gives `s` "
            "integer storage first and refuses the float update (newt/compiler/codegen.py:826-865)",
    },
}

_RUNNER = """
import sys
sys.path.insert(0, {root!r})
import newt_b200
newt_b200.install_aliases()
import pytest
sys.exit(pytest.main([{path!r}, "-q", "-rfE", "--no-header", "-p", "no:cacheprovider"]))
"""


def _reference_tests():
    base = os.environ.get("NEWT_REFERENCE_DIR")
    folder = os.path.join(base, "tests") if base else None
    return folder if folder and os.path.isdir(folder) else None


@pytest.mark.parametrize("name", FILES)
def test_reference_file(name, tmp_path):
    folder = _reference_tests()
    if folder is None:
        pytest.skip("NEWT_REFERENCE_DIR does not name a checkout of the reference")
    path = os.path.join(folder, name)
    if not os.path.exists(path):
        pytest.skip(f"{name} is not in that checkout")
    env = dict(os.environ, DEUTERON_CACHE_DIR=str(tmp_path / "deuteron"),
               NEWT_CACHE_DIR=str(tmp_path / "newt"))
    run = subprocess.run([sys.executable, "-c", _RUNNER.format(root=ROOT, path=path)],
                         capture_output=True, text=True, env=env, timeout=1500)
    text = run.stdout + run.stderr
    failed = re.findall(r"^(?:FAILED|ERROR) \S*?::(\S+)", text, flags=re.M)
    summary = text.strip().splitlines()[-1] if text.strip() else "(no output)"
    report = os.environ.get("NEWT_REFERENCE_REPORT")
    if report:
        with open(report, "a") as f:
            f.write(f"{name}: {summary}\n" + "".join(f"    {t}\n" for t in failed))
    unexpected = [t for t in failed if t not in KNOWN.get(name, {})]
    assert not unexpected, f"{name}: {summary}\n" + "\n".join(unexpected) + "\n" + text[-4000:]
    assert re.search(r"\d+ passed", summary) or failed, f"{name} collected nothing: {text[-2000:]}"
