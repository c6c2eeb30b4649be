"""Guards on the source tree: layering of the package, no tracing compilers or foreign kernel languages on the
execution path, no closed CUDA calls, comments that stand on their own."""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]
PKG = ROOT / "litevllm_b200"
SOURCES = [p for pat in ("*.py", "*.cu", "*.cuh", "*.h", "*.cpp") for top in (PKG, ROOT / "csrc", ROOT / "benchmarks", ROOT / "tests")
           for p in top.rglob(pat)] + [ROOT / "bench.py", ROOT / "__graft_entry__.py"]


def _imports(path: Path) -> list[str]:
    return re.findall(r"^\s*(?:from|import)\s+([.\w]+)", path.read_text(), flags=re.M)


def _imports_of(folder: str, *targets: str) -> list[str]:
    bad = []
    for p in (PKG / folder).rglob("*.py"):
        for mod in _imports(p):
            tail = mod.lstrip(".")
            if mod.startswith(".") and any(tail == t or tail.startswith(t + ".") for t in targets):
                bad.append(f"{p.relative_to(ROOT)}: {mod}")
            if any(mod.startswith(f"litevllm_b200.{t}") for t in targets):
                bad.append(f"{p.relative_to(ROOT)}: {mod}")
    return bad


def test_kernel_and_layer_code_does_not_reach_up_into_the_engine():
    assert _imports_of("ops", "engine", "entrypoints", "adapters", "models") == []
    assert _imports_of("layers", "engine", "entrypoints", "adapters") == []
    assert _imports_of("loaders", "engine", "entrypoints") == []
    for folder in ("engine", "parallel", "adapters", "config", "models", "layers", "ops"):
        assert _imports_of(folder, "entrypoints") == [], folder


def test_no_tracing_compiler_or_foreign_kernel_language_in_the_package():
    pat = re.compile(r"^\s*(?:import|from)\s+(triton|tilelang|jax)\b|torch\.compile\(|@triton\.jit|wgmma\.", re.M)
    hits = [str(p.relative_to(ROOT)) for p in SOURCES if p.is_relative_to(PKG) or p.is_relative_to(ROOT / "csrc")
            if pat.search(p.read_text())]
    assert hits == []


def test_closed_cuda_calls_and_cluster_multicast_loads_are_absent():
    closed = re.compile("|".join(["cuda" + "Memcpy" + "BatchAsync", "cuda" + "Memcpy3D" + "BatchAsync",
                                  "cu" + "Memcpy" + "BatchAsync", "cu" + "Memcpy3D" + "BatchAsync"]))
    multicast_load = re.compile(r"cp\.async\.bulk(?:\.tensor)?[.\w:]*\.multicast" + "::cluster")
    for p in SOURCES:
        if p == Path(__file__).resolve():
            continue
        text = p.read_text()
        assert not closed.search(text), p
        assert not multicast_load.search(text), p


def test_every_wait_in_a_kernel_has_a_limit():
    """A loop that polls a flag, a peer or a barrier counts its iterations; no bare ``while (true)`` / ``for (;;)``
    without a bound in sight, and no trap instruction."""
    for p in (ROOT / "csrc").rglob("*.cu*"):
        text = p.read_text()
        assert "__trap" not in text and "asm volatile(\"trap" not in text, p
        for m in re.finditer(r"while\s*\(\s*(?:true|1)\s*\)|for\s*\(\s*;\s*;\s*\)", text):
            window = text[m.start(): m.start() + 900]
            assert re.search(r"spins|iters?\b|tries|budget|limit|kMax|max_|clock64|globaltimer|break;|return", window), \
                f"{p.name}: unbounded loop near offset {m.start()}"


def test_comments_name_no_build_documents_or_machine_paths():
    words = re.compile(r"SURVEY|VERDICT|ADVICE\.md|DESIGN\.md|BASELINE\.md|gpu" + r"run|/ro" + r"ot/|\bjud" + r"ge\b|\bround \d")
    hits = []
    for p in SOURCES:
        if p == Path(__file__).resolve():
            continue
        for n, line in enumerate(p.read_text().splitlines(), 1):
            if words.search(line):
                hits.append(f"{p.relative_to(ROOT)}:{n}: {line.strip()[:80]}")
    assert hits == []


def test_every_test_needing_a_gpu_is_marked():
    for p in (ROOT / "tests").rglob("test_*.py"):
        text = p.read_text()
        for m in re.finditer(r"^def (test_\w+)\(", text, flags=re.M):
            name = m.group(1)
            if name.endswith("_gpu") or "_on_gpu" in name or "_on_the_gpu" in name:
                head = text[max(0, m.start() - 400): m.start()]
                assert "pytest.mark.gpu" in head or "pytestmark" in text, f"{p.name}::{name} lacks the gpu mark"


def test_the_regression_ladder_script_parses_and_names_existing_files():
    import subprocess
    script = ROOT / "tests" / "run_regression_suite.sh"
    assert subprocess.run(["bash", "-n", str(script)]).returncode == 0
    out = subprocess.run(["bash", str(script), "--help"], capture_output=True, text=True)
    assert out.returncode == 0 and "--gpu" in out.stdout
    assert subprocess.run(["bash", str(script), "--bogus"], capture_output=True).returncode == 2
    for name in re.findall(r"tests/test_\w+\.py", script.read_text()):
        assert (ROOT / name).is_file(), name
