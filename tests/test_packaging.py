"""The drop-in boundary as an installable distribution: the vLLM plugin entry point and the reference's
top-level import names (``nvfp4``, ``nvfp4.mxfp4``, ``nvfp4.cute_fold``, ``nvfp4.cute_attn``, ``quant``,
``residue_vllm_plugin``) are declared in pyproject.toml and resolve to this package."""
import os
import subprocess
import sys
import tomllib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _project():
    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as f:
        return tomllib.load(f)


def test_entry_point_and_package_map_are_declared():
    cfg = _project()
    eps = cfg["project"]["entry-points"]["vllm.general_plugins"]
    assert eps == {"residue_patch": "residue_vllm_plugin:apply"}       # runtime/vllm_plugin/pyproject.toml:16-19
    st = cfg["tool"]["setuptools"]
    for name in ("nvfp4", "quant", "residue_vllm_plugin", "resinfer_b200.nvfp4.mxfp4", "resinfer_b200.nvfp4.cute_fold",
                 "resinfer_b200.nvfp4.cute_attn", "resinfer_b200.runtime.vllm_plugin"):
        assert name in st["packages"]
    for name, rel in st["package-dir"].items():
        assert os.path.isfile(os.path.join(ROOT, rel, "__init__.py")), name
    for pkg in st["packages"]:
        if pkg.startswith("resinfer_b200"):
            assert os.path.isfile(os.path.join(ROOT, *pkg.split("."), "__init__.py")), pkg


def test_reference_import_names_resolve_to_this_package():
    """What an installed copy does, without installing: the hand-over packages first on the path."""
    code = (
        "import nvfp4, nvfp4.mxfp4, nvfp4.cute_fold.host, nvfp4.cute_attn.host, nvfp4.cute_attn.plan\n"
        "import quant.linear_registry, quant.vllm_integration.residue_tp\n"
        "import residue_vllm_plugin\n"
        "assert nvfp4.__name__ == 'resinfer_b200.nvfp4', nvfp4.__name__\n"
        "assert nvfp4.mxfp4.__name__ == 'resinfer_b200.nvfp4.mxfp4'\n"
        "assert nvfp4.cute_attn.host.__name__ == 'resinfer_b200.nvfp4.cute_attn.host'\n"
        "assert quant.linear_registry.LinearRegistry.__module__ == 'resinfer_b200.quant.linear_registry'\n"
        "assert residue_vllm_plugin.apply.__module__ == 'resinfer_b200.runtime.vllm_plugin.residue_vllm_plugin'\n"
        "print('ok')\n")
    env = dict(os.environ, PYTHONPATH=os.pathsep.join([os.path.join(ROOT, "resinfer_b200", "_compat"), ROOT]))
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, cwd="/", timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), r.stderr[-2000:]
