"""The reference-side binding, checked without a node runtime: the N-API shim
(torchlette_b200/csrc/napi/tl_napi.c) must compile cleanly, must export one function per entry
point of include/tlcuda.h, and -- linked against a fake N-API and fakes of the C ABI
(tests/napi_stub/stub_napi.c) -- must hand the library the right byte counts for subarray
views, the right shape count to tl_pretune, the epilogue's ops and inputs, free device memory
exactly once from finalizers, and settle downloadAsync's Promise only after its work item ran."""
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "torchlette_b200", "csrc", "napi", "tl_napi.c")
STUB = os.path.join(ROOT, "tests", "napi_stub", "stub_napi.c")
HEADER = os.path.join(ROOT, "include", "tlcuda.h")
INC = os.path.join(ROOT, "include")


def _header_exports():
    text = open(HEADER).read()
    return re.findall(r"^TL_API\s+[\w\s\*]+?\b(tl_\w+)\s*\(", text, flags=re.M)


def _camel(c_name):
    parts = c_name[len("tl_"):].split("_")
    return parts[0] + "".join(p[:1].upper() + p[1:] for p in parts[1:])


def test_shim_compiles_without_warnings():
    subprocess.run(["gcc", "-std=c11", "-fsyntax-only", "-Wall", "-Wextra", "-Werror", "-I", INC, SHIM], check=True)


@pytest.fixture(scope="module")
def harness(tmp_path_factory):
    exe = str(tmp_path_factory.mktemp("napi") / "napi_stub_test")
    subprocess.run(["gcc", "-std=c11", "-Wall", "-Wextra", "-Werror", "-O1", "-no-pie", "-I", INC, SHIM, STUB,
                    "-Wl,--unresolved-symbols=ignore-all", "-o", exe], check=True)
    return exe


def test_every_header_function_has_an_export(harness):
    names = _header_exports()
    assert len(names) >= 68
    exported = set(subprocess.run([harness, "--list"], check=True, capture_output=True, text=True).stdout.split())
    shim_text = open(SHIM).read()
    missing = [n for n in names if _camel(n) not in exported or not re.search(r"\b%s\b" % n, shim_text)]
    assert not missing, f"no N-API export for: {missing}"


def test_shim_behaviour_against_fake_napi(harness):
    r = subprocess.run([harness], capture_output=True, text=True)
    assert r.returncode == 0 and r.stdout.strip().endswith("ALL OK"), r.stdout + r.stderr
    for line in ("ok upload copies the view's own 16 bytes", "ok pretune passes 2 shapes and the descriptor",
                 "ok downloadAsync resolves with the filled view and frees its staging",
                 "ok a dropped owning buffer is freed once by its finalizer"):
        assert line in r.stdout


def test_integration_patch_applies_to_a_reference_checkout(tmp_path):
    """integration/torchlette.diff against a torchlette checkout named by TORCHLETTE_REFERENCE
    (skipped when the variable is unset): `patch --dry-run` must accept every hunk."""
    ref = os.environ.get("TORCHLETTE_REFERENCE")
    if not ref or not os.path.isdir(ref):
        pytest.skip("TORCHLETTE_REFERENCE does not name a checkout")
    patch = os.path.join(ROOT, "integration", "torchlette.diff")
    files = re.findall(r"^\+\+\+ b/(\S+)", open(patch).read(), flags=re.M)
    assert files
    for f in files:
        dst = tmp_path / f
        dst.parent.mkdir(parents=True, exist_ok=True)
        dst.write_bytes(open(os.path.join(ref, f), "rb").read())
    subprocess.run(["patch", "-p1", "--dry-run", "-i", patch], cwd=tmp_path, check=True, capture_output=True)
