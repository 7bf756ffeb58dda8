"""baseline/vendor_reference.py: the one documented edit of transformer/model.py is verified line by line, and a
checkout whose lines differ is refused."""
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _module():
    spec = importlib.util.spec_from_file_location("vendor_reference", os.path.join(ROOT, "baseline", "vendor_reference.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_edits_are_three_lines_inside_the_attention_block():
    mod = _module()
    assert sorted(mod.EDITS) == [292, 293, 300]
    for old, new in mod.EDITS.values():
        assert old.strip().split(" = ")[0] == new.strip().split(" = ")[0]      # same variable, new right-hand side
        assert new.strip().split(" = ")[1].startswith("self.")


def test_a_checkout_with_different_lines_is_refused(tmp_path):
    mod = _module()
    ref = tmp_path / "ref"
    (ref / "transformer").mkdir(parents=True)
    (ref / "attention_mechanisms").mkdir()
    (ref / "transformer" / "model.py").write_text("\n" * 400)
    (ref / "transformer" / "modules.py").write_text("import kornia\n")
    with pytest.raises(RuntimeError):
        mod.vendor(str(ref))
    with pytest.raises(FileNotFoundError):
        mod.vendor(str(tmp_path / "nowhere"))
