"""Link-level half of the drop-in proof, no GPU: every symbol the C callers and the reference's
scheduler import from the model library is one this repository's library exports."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DROP = os.path.join(ROOT, "oracle", "_ref", "dropin")
LIB = os.path.join(ROOT, "s2pro-native_b200", "libs2pro_b200.so")


def symbols(path, flag):
    out = subprocess.run(["nm", "-D", flag, path], capture_output=True, text=True, check=True).stdout
    return {line.split()[-1].split("@")[0] for line in out.splitlines() if line.strip()}


@pytest.mark.parametrize("binary", ["model_caller_mine", "sched_caller_mine"])
def test_callers_import_only_exported_entry_points(binary):
    path = os.path.join(DROP, binary)
    if not (os.path.exists(path) and os.path.exists(LIB)):
        pytest.skip("drop-in callers not built on this machine")
    wanted = {s for s in symbols(path, "--undefined-only") if s.startswith("s2p_")}
    assert wanted, "the caller imports nothing from the model library"
    missing = wanted - symbols(LIB, "--defined-only")
    assert not missing, f"not exported by this library: {sorted(missing)}"
    # the binary names the library by its soname and finds it relative to itself
    dyn = subprocess.run(["readelf", "-d", path], capture_output=True, text=True, check=True).stdout
    assert "libs2pro_b200.so" in dyn and "$ORIGIN" in dyn


def test_both_binaries_of_a_pair_share_one_object_file():
    """The pair differs in the library it was linked with, not in the caller: same imported s2p_* set."""
    for stem in ("model_caller", "sched_caller"):
        a, b = (os.path.join(DROP, f"{stem}_{w}") for w in ("mine", "ref"))
        if not (os.path.exists(a) and os.path.exists(b)):
            pytest.skip("drop-in callers not built on this machine")
        sa = {s for s in symbols(a, "--undefined-only") if s.startswith("s2p_")}
        sb = {s for s in symbols(b, "--undefined-only") if s.startswith("s2p_")}
        assert sa == sb
