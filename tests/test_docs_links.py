"""Documentation lint: every repository path that the user-facing documents name in backticks exists.

The reference checks the links of its documents (experiments/bench/linkcheck.sh); the documents here
name files rather than URLs, so the check is on paths: a renamed kernel file or a removed profile
summary must not stay behind in README / docs / profiles.
"""
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
DOCUMENTS = [ROOT / "README.md", *sorted((ROOT / "docs").glob("*.md")), *sorted((ROOT / "profiles").glob("*.md")),
             ROOT / "repro" / "README.md"]
PREFIXES = ("aboleth_b200/", "tests/", "benchmarks/", "examples/", "docs/", "profiles/", "baseline/", "repro/",
            "csrc/", "include/")
# Paths inside the package are often written relative to it.
PACKAGE_RELATIVE = ("csrc/", "include/")


def _candidates(text: str):
    for quoted in re.findall(r"`([^`\n]+)`", text):
        for token in re.split(r"[\s,;]+", quoted):
            token = token.strip("()[]{}:.'\"")
            token = token.split("::")[0]                  # tests/x.py::test_name
            token = re.sub(r":\d+(-\d+)?$", "", token)      # file.py:10-20
            if token.startswith(PREFIXES) and not any(c in token for c in "*<>{}$|") and "..." not in token:
                yield token


def _bare_names(text: str):
    """File names written without a directory (`moe_kernels.cu`, `tp_fused_event_timings.md`)."""
    for quoted in re.findall(r"`([^`\n]+)`", text):
        for token in re.split(r"[\s,;]+", quoted):
            token = re.sub(r":\d+(-\d+)?$", "", token.strip("()[]{}:.'\"").split("::")[0])
            if re.fullmatch(r"[A-Za-z0-9_]+\.(py|cu|cuh|h|hpp|cpp|md)", token):
                yield token


def test_paths_named_in_the_documents_exist():
    missing = []
    for document in DOCUMENTS:
        for token in _candidates(document.read_text()):
            if "/_lib" in token:
                continue                                   # built artefacts, absent before the first build
            path = ROOT / ("aboleth_b200/" + token if token.startswith(PACKAGE_RELATIVE) else token)
            if token.endswith("/"):
                ok = path.is_dir()
            else:
                ok = path.exists() or path.with_suffix("").is_dir()
            if not ok:
                missing.append(f"{document.relative_to(ROOT)}: {token}")
    assert not missing, "stale paths:\n" + "\n".join(sorted(set(missing)))


def test_file_names_written_without_a_directory_exist_somewhere():
    tracked = {p.name for p in ROOT.rglob("*") if p.is_file() and "_work" not in p.parts
               and "gpurun_out" not in p.parts and ".git" not in p.parts}
    # Names of the reference's files and of files a command line creates are not ours to find.
    foreign = {"device.cuh"} - tracked
    missing = []
    for document in DOCUMENTS:
        text = document.read_text()
        for name in _bare_names(text):
            if name in tracked or name in foreign:
                continue
            # a sentence that cites the reference names its path in the same backticks or nearby
            if re.search(r"(python/aboleth|experiments/|integrations/vllm|include/aboleth/Target)[^`]*" + re.escape(name), text):
                continue
            missing.append(f"{document.relative_to(ROOT)}: {name}")
    assert not missing, "file names that exist nowhere in the repository:\n" + "\n".join(sorted(set(missing)))
