"""The public names a user of the reference package expects exist (no GPU)."""
import pytest

import aboleth_b200 as ab

EXPECTED = """AllocationHandle AllocationProvider Artifact AutoTransportPolicy Bootstrap CapacityContract CommunicationDataflow
CommunicationDataflowOperation CommunicationRegion CommunicationStage CompiledExecutionPlan CompiledKVCacheMigrationPlan
CompiledPattern CompiledPatternPlan CompiledPhase DeviceLibrary Endpoint EndpointMesh EndpointPair EndpointTable
ExecutionContract ExecutionDecision ExecutionFallback FragmentArtifact GENERIC_KV_TARGET_PROFILE
H200_NVLINK_KV_TARGET_PROFILE InvokeManifest KVCacheLayoutContract KVCacheMigrationSpec KVCachePhysicalization
KVRuntimeOverrides KVTargetProfile KernelBinding KernelTransportReduction LocalBuffer LocalEndpoint LocalRegion
MoEPatternSpec OpaqueCapabilities OpaqueStage OutputLifetimePlan P2PRealizationProfile PaddingSemantics Pattern
PeerRegionTable PhaseBinding PhaseResources PhaseSchedule PhysicalizedPattern PipeBootstrap PipeBootstrapCoordinator
RegionEffect RegionRequirement RankControl RegisteredBuffer RemoteBuffer RemoteHandle Runtime RuntimeGuard
RuntimeBindings RuntimeBufferBinding SimplifiedCommunicationDataflow StandaloneKernel TcpStoreBootstrap
TorchDistributedBootstrap Transport TransportKernel TransportPhase TransportPlan Workset World
build_kv_cache_migration_pattern build_moe_pattern compilation compile_execution_plan compile_fragment_artifact
compile_kv_cache_migration compile_phase connection_info_from_bytes connection_transport device_library drain
install_compiler invoke_transport_program physicalize_pattern plan_output_lifetimes plan_transport
plan_transport_facts plan_transport_program planned_wait put realize_bindable_epilogue realize_standalone_kernel
select_kv_target_profile signal simplify_communication_dataflow token token_type wait wait_signal""".split()


def test_reference_names_exist():
    missing = [name for name in EXPECTED if not hasattr(ab, name)]
    assert not missing, missing


def test_subpackages_import():
    import aboleth_b200.compiler  # noqa: F401
    import aboleth_b200.integrations  # noqa: F401
    import aboleth_b200.kv  # noqa: F401
    import aboleth_b200.models  # noqa: F401
    import aboleth_b200.moe  # noqa: F401
    import aboleth_b200.records  # noqa: F401
    from aboleth_b200.device_library import cached_device_library
    from aboleth_b200.integrations import AbolethAll2AllManager, AbolethPrepareAndFinalize  # noqa: F401
    from aboleth_b200.moe import MoESpec, NativeMoEFamily, NativeMoESlot, compile_moe_plan  # noqa: F401
    assert callable(cached_device_library)


def test_device_library_package(tmp_path, monkeypatch):
    import json
    import subprocess

    monkeypatch.setenv("ABOLETH_CACHE_DIR", str(tmp_path))
    lib = ab.device_library(transports=["p2p", "rdma"])
    manifest = json.loads(lib.manifest.read_text())
    assert manifest["abi"] == 2 and manifest["served_by_host_proxy"] == ["rdma"] and manifest["bounded_waits"]
    assert "put_many_signal" in manifest["operations"] and lib.header.exists()
    assert ab.device_library(transports=["p2p", "rdma"]).digest == lib.digest  # cache hit
    # A client kernel written against the facade compiles for sm_100a with the published flags.
    src = tmp_path / "client.cu"
    src.write_text('#include "aboleth/device.cuh"\n'
                   '__global__ void k(const std::uint64_t* eps, unsigned long long* st, '
                   'unsigned long long dst, unsigned long long src, unsigned long long flag) {\n'
                   '  aboleth::DeviceContext ctx{eps, nullptr, st};\n'
                   '  aboleth::put(ctx, 1, aboleth::RemoteRegion{dst, 0}, aboleth::LocalRegion{src, 0}, 256);\n'
                   '  aboleth::put_inline(ctx, 1, aboleth::RemoteRegion{dst + 256, 0}, 7);\n'
                   '  aboleth::signal(ctx, 1, aboleth::RemoteRegion{flag, 0}, 1);\n'
                   '  aboleth::quiet(ctx, 1);\n'
                   '  aboleth::wait_signal(ctx, (const std::uint64_t*)flag, 1);\n}\n')
    subprocess.run(["nvcc", *lib.nvcc_flags(), "-c", str(src), "-o", str(tmp_path / "client.o")], check=True)
    special = ab.device_library(transports=["p2p"], specialize="p2p")
    assert "ABOLETH_TIER1_SPECIALIZED" in special.header.read_text()


def test_device_library_archive_links_into_a_client(tmp_path, monkeypatch):
    """The static archive exports aboleth_tier1_<op>_<transport>; a client that only declares the
    symbols compiles with -rdc=true and links against it (device link included)."""
    import json
    import subprocess

    monkeypatch.setenv("ABOLETH_CACHE_DIR", str(tmp_path))
    lib = ab.device_library(transports=["p2p", "rdma"], archive=True)
    manifest = json.loads(lib.manifest.read_text())
    assert lib.archive is not None and lib.archive.exists() and not manifest["header_only"]
    assert "aboleth_tier1_put_signal_p2p" in manifest["symbols"] and "aboleth_tier1_quiet_rdma" in manifest["symbols"]
    assert ab.device_library(transports=["p2p", "rdma"], archive=True).archive == lib.archive  # cache hit
    src = tmp_path / "client.cu"
    src.write_text('extern "C" __device__ unsigned long long aboleth_tier1_put_signal_p2p(unsigned long long, unsigned, '
                   'unsigned long long, unsigned, unsigned long long, unsigned, unsigned, unsigned long long, unsigned, '
                   'unsigned long long);\n'
                   'extern "C" __device__ unsigned long long aboleth_tier1_wait_signal(unsigned long long, '
                   'unsigned long long, unsigned long long);\n'
                   '__global__ void k(unsigned long long eps, unsigned long long dst, unsigned long long src, '
                   'unsigned long long flag, unsigned long long *status) {\n'
                   '  status[0] = aboleth_tier1_put_signal_p2p(eps, 1, dst, 0, src, 0, 256, flag, 0, 1);\n'
                   '  status[1] = aboleth_tier1_wait_signal(flag, 1, 1000000);\n}\n'
                   'int main() { return 0; }\n')
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-rdc=true", str(src),
                    f"-L{lib.archive.parent}", "-laboleth_tier1", "-o", str(tmp_path / "client")], check=True)


def test_device_library_lanes_and_compile_time_peers(tmp_path, monkeypatch):
    import subprocess

    monkeypatch.setenv("ABOLETH_CACHE_DIR", str(tmp_path))
    lib = ab.device_library(transports=["p2p"], endpoints_per_peer=4)
    text = lib.header.read_text()
    assert "#define ABOLETH_TIER1_ENDPOINTS_PER_PEER 4" in text and "#define ABOLETH_TIER1_SMALL_INLINE 1" in text
    src = tmp_path / "lanes.cu"
    src.write_text('#include "aboleth/device.cuh"\n'
                   'static_assert(aboleth::kEndpointsPerPeer == 4, "lanes");\n'
                   '__global__ void k(const std::uint64_t* eps, unsigned long long* st, unsigned long long dst, '
                   'unsigned long long src, unsigned long long flag) {\n'
                   '  aboleth::DeviceContext ctx{eps, nullptr, st};\n'
                   '  aboleth::put_signal<1>(ctx, aboleth::RemoteRegion{dst, 0}, aboleth::LocalRegion{src, 0}, 64, '
                   'aboleth::RemoteRegion{flag, 0}, 1);\n'
                   '  aboleth::put_inline_small(ctx, aboleth::open(ctx, 2), aboleth::RemoteRegion{dst, 0}, 0x010203, 3);\n'
                   '  aboleth::quiet<1>(ctx);\n}\n')
    subprocess.run(["nvcc", *lib.nvcc_flags(), "-c", str(src), "-o", str(tmp_path / "lanes.o")], check=True)


def test_extern_symbol_table_and_prototype_header_link(tmp_path, monkeypatch):
    """The language-neutral binding: a client that includes nothing but the generated prototypes
    calls every exported symbol and links against the archive."""
    import subprocess

    from aboleth_b200 import frontends

    monkeypatch.setenv("ABOLETH_CACHE_DIR", str(tmp_path))
    transports = ["p2p", "proxy"]
    table = frontends.extern_symbols(transports)
    names = [s.name for s in table]
    assert len(names) == len(set(names)) == 2 * 8 + 1 and names[-1] == "aboleth_tier1_wait_signal"
    put_signal = next(s for s in table if s.name == "aboleth_tier1_put_signal_proxy")
    assert put_signal.arg_types == ("u64", "u32", "u64", "u32", "u64", "u32", "u32", "u64", "u32", "u64")
    assert put_signal.arg_names[:2] == ("endpoints", "peer") and put_signal.return_type == "u64"
    with pytest.raises(ValueError, match="unknown transports"):
        frontends.extern_symbols(["gin"])

    lib = ab.device_library(transports=transports, archive=True)
    import json
    assert set(names) == set(json.loads(lib.manifest.read_text())["symbols"])  # the table is the archive's
    header = frontends.write_prototypes(lib, transports)
    calls = []
    for symbol in table:
        args = ", ".join("a" if t == "u64" else "b" for t in symbol.arg_types)
        calls.append(f"  s += {symbol.name}({args});")
    src = tmp_path / "client.cu"
    src.write_text(f'#include "aboleth/{header.name}"\n'
                   "__global__ void k(unsigned long long a, unsigned b, unsigned long long *out) {\n"
                   "  unsigned long long s = 0;\n" + "\n".join(calls) + "\n  *out = s;\n}\nint main() { return 0; }\n")
    subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", *frontends.link_flags(lib), str(src),
                    "-o", str(tmp_path / "client")], check=True)
    with pytest.raises(ValueError, match="header-only"):
        frontends.link_flags(ab.device_library(transports=["p2p"]))


def test_specialised_library_pins_its_transport_at_compile_time(tmp_path):
    """A library specialised for peer memory compiles peer-memory clients, says so in its macros, and
    refuses - at compile time - code written for the host ring (reference: docs/TIERS.md:52-66)."""
    import shutil
    import subprocess

    from aboleth_b200.device_library import generate_device_library

    nvcc = shutil.which("nvcc")
    if nvcc is None:
        pytest.skip("needs nvcc")
    lib = generate_device_library(tmp_path / "p2p", transports=["p2p"], specialize="p2p")
    text = lib.header.read_text()
    assert "#define ABOLETH_TIER1_GENERATED 1" in text and "#define ABOLETH_TIER1_SPECIALIZED 1" in text
    client = tmp_path / "client.cu"
    body = '''#include "aboleth/device.cuh"
static_assert(ABOLETH_TIER1_GENERATED == 1 && ABOLETH_TIER1_HAS_P2P == 1 && ABOLETH_TIER1_HAS_PROXY == 0, "macros");
static_assert(aboleth::kServes<aboleth::abi::kKindP2P> && !aboleth::kServes<aboleth::abi::kKindProxy>, "kinds");
__global__ void k(const std::uint64_t *eps, unsigned long long dst, unsigned long long src, unsigned long long flag) {
    aboleth::DeviceContext ctx{eps, nullptr};
    const aboleth::PeerRef ref = aboleth::open_as<aboleth::abi::%s>(ctx, 1);
    aboleth::put_signal(ctx, ref, aboleth::RemoteRegion{dst, 0}, aboleth::LocalRegion{src, 0}, 64,
                        aboleth::RemoteRegion{flag, 0}, 1);
}
'''
    compile_cmd = [nvcc, *lib.nvcc_flags(), "-c", str(client), "-o", str(tmp_path / "client.o")]
    client.write_text(body % "kKindP2P")
    assert subprocess.run(compile_cmd, capture_output=True, text=True).returncode == 0
    client.write_text((body % "kKindProxy").replace("ABOLETH_TIER1_HAS_PROXY == 0", "true"))
    refused = subprocess.run(compile_cmd, capture_output=True, text=True)
    assert refused.returncode != 0 and "specialised for another transport" in refused.stderr
    # the tree's own header is the unspecialised, not-generated form
    unspecialised = generate_device_library(tmp_path / "both", transports=["p2p", "proxy"])
    assert "#define ABOLETH_TIER1_SPECIALIZED" not in unspecialised.header.read_text().split("#ifdef ABOLETH_TIER1_SPECIALIZED")[0]
    with pytest.raises(ValueError, match="none of the requested transports"):
        generate_device_library(tmp_path / "bad", transports=["p2p"], specialize="proxy")


def test_pinned_environment_check_reports_every_pin(tmp_path):
    from pathlib import Path

    """The checker names each pinned package with what it found; a wrong pin of a required package
    fails, a wrong pin of a baseline-only package only warns."""
    import json

    from aboleth_b200.utils import environment

    pins = json.loads((Path(__file__).resolve().parent.parent / "repro" / "environment.json").read_text())
    result = environment.compare(pins)
    names = [row[0] for row in result["rows"]]
    assert set(pins["packages"]) <= set(names) and "python" in names and "nvcc" in names
    assert all(row[3] in ("ok", "warn", "fail") for row in result["rows"])
    wrong = dict(pins, packages={**pins["packages"], "torch": "0.0.0"})
    assert environment.compare(wrong)["ok"] is False
    only_baseline = dict(pins, packages={**pins["packages"], "vllm": "0.0.0"})
    rows = {row[0]: row[3] for row in environment.compare(only_baseline)["rows"]}
    assert rows["vllm"] == "warn"


def test_every_benchmark_preset_builds_a_runnable_command():
    """Each preset names a script that exists and flags that the script's parser knows; multi-rank presets go
    through torchrun on 127.0.0.1."""
    import importlib.util
    import re
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    spec = importlib.util.spec_from_file_location("bench_run", root / "benchmarks" / "run.py")
    run = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(run)
    for name, (script, extra, allowed, what) in run.PRESETS.items():
        assert what and allowed
        gpus = max(allowed)
        command = run.command(name, gpus, Path("out"), 29600)
        if script.startswith("-m"):
            continue
        path = (root / "benchmarks" / script).resolve()
        assert path.exists(), (name, path)
        source = path.read_text()
        for flag in [a for a in extra if a.startswith("--")] + (["--out"] if name != "headline" else []):
            assert re.search(r'"%s"' % re.escape(flag), source), (name, flag)
        if gpus > 1 and name not in ("native", "nccl-host", "peer-copy"):
            assert "torch.distributed.run" in command and "127.0.0.1" in command
