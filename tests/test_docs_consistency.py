"""What the documentation names must exist: modules, settings and command-line flags."""
import importlib.util
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DOCS = [os.path.join(ROOT, "README.md")] + sorted(
    os.path.join(ROOT, "docs", f) for f in os.listdir(os.path.join(ROOT, "docs")) if f.endswith(".md"))


def texts():
    for path in DOCS:
        with open(path) as fh:
            yield os.path.relpath(path, ROOT), fh.read()


def source_text() -> str:
    chunks = []
    for base, dirs, files in os.walk(os.path.join(ROOT, "gpubridge_b200")):
        dirs[:] = [d for d in dirs if d not in ("_build", "lib", "__pycache__")]
        for name in files:
            if name.endswith((".py", ".cu", ".cuh", ".cpp", ".h", ".sh", ".sbatch")):
                with open(os.path.join(base, name), errors="replace") as fh:
                    chunks.append(fh.read())
    for name in ("bench.py", "tests/conftest.py"):
        with open(os.path.join(ROOT, name)) as fh:
            chunks.append(fh.read())
    return "\n".join(chunks)


def resolves(dotted: str) -> bool:
    """``a.b.c`` names a module, or an attribute of the longest module prefix."""
    parts = dotted.split(".")
    for cut in range(len(parts), 0, -1):
        name = ".".join(parts[:cut])
        try:
            if importlib.util.find_spec(name) is None:
                continue
        except (ImportError, AttributeError, ValueError):
            continue
        if cut == len(parts):
            return True
        obj = importlib.import_module(name)
        for attr in parts[cut:]:
            if not hasattr(obj, attr):
                return False
            obj = getattr(obj, attr)
        return True
    return False


def test_named_modules_exist():
    missing = []
    for path, text in texts():
        for module in set(re.findall(r"gpubridge_b200(?:\.[a-z_][a-z_0-9]*)+", text)):
            if not resolves(module.rstrip(".")):
                missing.append((path, module))
        for short in set(re.findall(r"`(?:bench|kit)\.([a-z_][a-z_0-9]*)", text)) - {"py"}:
            if not any(resolves(f"gpubridge_b200.{pkg}.{short}") for pkg in ("bench", "kit")):
                missing.append((path, short))
    assert not missing, missing


def test_named_settings_exist():
    source = source_text()
    unknown = sorted({name for _, text in texts() for name in re.findall(r"GPUBRIDGE_[A-Z0-9_]+", text)
                      if name not in source})
    # settings of the reference that this build does not read are named in the migration notes only
    assert not unknown, unknown


def test_named_flags_exist():
    source = source_text()
    with open(os.path.join(ROOT, "examples", "fsdp2_torch_backend.py")) as fh:
        source += fh.read()
    unknown = sorted({flag for _, text in texts() for flag in re.findall(r"`(--[a-z][a-z0-9-]+)", text)
                      if f'"{flag}"' not in source and flag not in ("--nproc-per-node", "--gres", "--gpus")})
    assert not unknown, unknown
