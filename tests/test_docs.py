"""The API reference names every method and op the native library binds, and every option the
runtime accepts - so a binding added without documentation fails here, on CPU."""
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parent.parent


def test_api_reference_names_every_bound_method_and_op():
    binding = (ROOT / "csrc" / "binding.cpp").read_text()
    names = set(re.findall(r'def\("([a-z_0-9]+)"', binding))
    assert len(names) > 30
    api = (ROOT / "docs" / "api.md").read_text()
    missing = sorted(n for n in names if f"`{n}" not in api and f"{n}(" not in api)
    assert not missing, missing


def test_api_reference_names_every_option():
    impl = (ROOT / "csrc" / "runtime" / "overlap_impl.cpp").read_text()
    options = set(re.findall(r'name == "([a-z_0-9]+)"', impl))
    assert {"mode", "stage_local", "timeout_ms"} <= options
    api = (ROOT / "docs" / "api.md").read_text()
    missing = sorted(o for o in options if f"`{o}`" not in api)
    assert not missing, missing
