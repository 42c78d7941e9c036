"""The drop-in boundary on a machine without a GPU: libmacllm_b200.so loads, exports every function the public header
declares, the ctypes mirror binds exactly that set, and the structs the two sides exchange have the same size and
field offsets (the header is compiled with gcc to ask the C side)."""
import ctypes as C
import importlib
import re
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
HEADER = ROOT / "include" / "macllm_b200.h"

STRUCTS = {
    "mk_load_config": "LoadConfig", "mk_runtime_spec": "RuntimeSpec", "mk_kv_capacity": "KvCapacity", "mk_pool_stats": "PoolStats",
    "mk_prefix_diagnostics": "PrefixDiagnostics", "mk_lane": "Lane", "mk_engine_config": "EngineConfig", "mk_request": "Request",
    "mk_tick_lane": "TickLane", "mk_engine_stats": "EngineStats", "mk_kernel_profile": "KernelProfile", "mk_attn_case": "AttnCase",
    "mk_gguf_summary": "GgufSummary", "mk_lane_sampling": "LaneSampling", "mk_tick_info": "TickInfo", "mk_batch_trace": "BatchTrace", "mk_request_metrics": "RequestMetrics",
}


def declared_functions():
    text = re.sub(r"/\*.*?\*/", "", HEADER.read_text(), flags=re.S)
    return sorted(set(re.findall(r"^\s*(?:const\s+)?[A-Za-z_0-9]+\s*\*?\s*(mk_[a-z0-9_]+)\s*\(", text, flags=re.M)))


@pytest.fixture(scope="module")
def capi(mk):
    return importlib.import_module("macllm_infer_b200._capi")


def test_library_exports_every_declared_function(capi):
    names = declared_functions()
    assert len(names) > 60 and "mk_model_load_gguf" in names and "mk_model_ep_init" in names
    handle = C.CDLL(str(capi.LIB_PATH))
    missing = [n for n in names if not hasattr(handle, n)]
    assert missing == []


def test_python_mirror_binds_exactly_the_declared_functions(capi):
    assert sorted(capi.SIGNATURES) == declared_functions()


def test_struct_layouts_match_the_header(capi, tmp_path):
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{HEADER}"', "int main(void) {"]
    for cname, pyname in STRUCTS.items():
        cls = getattr(capi, pyname)
        lines.append(f'printf("{cname} %zu", sizeof({cname}));')
        for field, _ in cls._fields_:
            lines.append(f'printf(" %zu", offsetof({cname}, {field}));')
        lines.append('printf("\\n");')
    lines += ["return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run(["gcc", "-std=c11", "-o", str(exe), str(src)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout.strip().splitlines()
    assert len(out) == len(STRUCTS)
    for line in out:
        cname, size, *offsets = line.split()
        cls = getattr(capi, STRUCTS[cname])
        assert C.sizeof(cls) == int(size), cname
        assert [getattr(cls, f).offset for f, _ in cls._fields_] == list(map(int, offsets)), cname
    # every struct with a body in the header is covered
    text = HEADER.read_text()
    assert sorted(re.findall(r"typedef struct (mk_[a-z_]+) \{", text)) == sorted(STRUCTS)


def test_expert_parallel_init_is_refused_on_a_host_only_model(capi):
    eng = importlib.import_module("macllm_infer_b200.engine")
    model = eng.Model.fake(vocab=32, max_context=64, kv_capacity_tokens=256)
    with pytest.raises(capi.MkError, match="GGUF model"):
        model.ep_init(bytes(128))
    with pytest.raises(ValueError):
        model.ep_init(bytes(5))
