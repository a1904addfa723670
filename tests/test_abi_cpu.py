"""CPU-only checks of the boundary: the shared library loads, exports exactly what
include/llama_rust_b200.h declares, and its host-only entry points behave."""
import ctypes as C
import glob
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from llama_rust_b200 import build, executor
    build.build()
    return executor.lib()


def declared_symbols():
    names = set()
    for h in glob.glob(os.path.join(ROOT, "include", "*.h")):
        text = re.sub(r"/\*.*?\*/", "", open(h).read(), flags=re.S)
        names |= set(re.findall(r"\b(llr_[a-z0-9_]+)\s*\(", text))
    return sorted(names)


def test_library_exports_every_declared_symbol(lib):
    from llama_rust_b200 import _lib
    declared = declared_symbols()
    assert declared, "no declarations found"
    for name in declared:
        assert hasattr(lib, name), f"{name} declared in include/ but not exported"
    assert sorted(_lib.SYMBOLS) == declared


def test_row_bytes_matches_reference_table(lib, orc):
    from llama_rust_b200 import executor as ex
    for kind in (0, 1, 2, 5, 6, 7, 12, 13, 17, 18, 19):
        for cols in (0, 256, 4096, 14336):
            assert ex.row_bytes(kind, cols) == orc.row_bytes(kind, cols)
    # benchmark shapes (quant.rs:86-163)
    assert ex.row_bytes(13, 4096) == 4352 and ex.row_bytes(17, 4096) == 2304
    assert ex.row_bytes(17, 14336) == 8064 and ex.row_bytes(19, 4096) == 3360
    assert ex.row_bytes(19, 14336) == 11760 and ex.row_bytes(6, 4096) == 2816 and ex.row_bytes(7, 4096) == 3072
    with pytest.raises(ex.NativeCudaError) as e:
        ex.row_bytes(13, 33)
    assert e.value.code == ex.ERR_UNALIGNED
    assert ex.row_bytes(5, 4096) == 2560 and ex.row_bytes(18, 4096) == 2816
    for bad in (3, 4, 8, 14, 16, 20, 255):  # the other GemmKind tags are out of scope
        with pytest.raises(ex.NativeCudaError) as e:
            ex.row_bytes(bad, 256)
        assert e.value.code == ex.ERR_DTYPE


def test_executor_creation_fails_loudly_without_a_gpu(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    from llama_rust_b200 import executor as ex
    with pytest.raises(ex.NativeCudaError) as e:
        ex.Executor(0)
    assert e.value.code in (ex.ERR_CUDA, ex.ERR_INVALID)
    assert str(e.value)


def test_null_handles_are_rejected(lib):
    assert lib.llr_exec_destroy(None) == 0
    assert lib.llr_matrix_free(None) == 0
    out = C.c_size_t()
    assert lib.llr_exec_mem_info(None, C.byref(out), C.byref(out)) != 0
    assert lib.llr_matmul(None, 13, 1, 32, 1, None, 34, None, 32, None, 1) != 0


def test_host_synth_is_deterministic_and_well_formed(orc):
    from llama_rust_b200 import synth
    a = synth.packed_matrix(synth.Q4_K, 8, 512, 99)
    b = synth.packed_matrix(synth.Q4_K, 8, 512, 99)
    assert np.array_equal(a, b) and a.size == 8 * 2 * 144
    assert not np.array_equal(a, synth.packed_matrix(synth.Q4_K, 8, 512, 100))
    # a block is independent of where the chunk boundaries fall
    assert np.array_equal(synth.packed_blocks(synth.Q6_K, 5, 3, 7), synth.packed_matrix(synth.Q6_K, 1, 2048, 7)[5 * 210:8 * 210])
    q = synth.packed_matrix(synth.Q8_0, 4, 256, 1).reshape(-1, 34)[:, 2:].view(np.int8)
    assert q.min() >= -127 and q.max() <= 127
    w = orc.dequant_matrix(orc.Q4_K, 8, 512, a)
    assert np.all(np.isfinite(w))
    x = synth.activations(4096, 3)
    assert abs(float(x.mean())) < 0.1 and 0.9 < float(x.std()) < 1.1
    assert synth.tensor_seed(0, "blk.0.attn_q.weight") != synth.tensor_seed(0, "blk.1.attn_q.weight")


def test_plan_placement_follows_the_byte_volume_rule():  # expertvm/src/tests.rs:441-454, planner.rs:332-349
    from llama_rust_b200 import DISPATCH_ACTIVATIONS, MOVE_WEIGHTS, plan_placement
    expert, act, pcie = 188 << 20, 4096, 32 * 1_000_000_000
    assert plan_placement(expert, act, 1, 1, pcie) == DISPATCH_ACTIVATIONS
    assert plan_placement(expert, act, 1, 64_000, pcie) == MOVE_WEIGHTS
    assert plan_placement(expert, act, 0, 0, pcie) == DISPATCH_ACTIVATIONS      # zero fan-in and reuse count as one
    assert plan_placement(4096, 4096, 1, 1, pcie) == MOVE_WEIGHTS               # a tie moves the weights
    assert plan_placement(expert, act, 1, 1, 0) == MOVE_WEIGHTS                 # no link: both infinite, tie
    assert plan_placement(1 << 40, 1 << 40, 1 << 40, 1 << 40, 1) == MOVE_WEIGHTS  # saturating products


def test_expert_parallel_arena_size_covers_both_halves_of_the_exchange():
    """llr_moe_ep_arena_bytes is host arithmetic: per half of the double-buffered arena, one receive slot of n_embd floats
    (plus a row tag) for every (local expert, sender, position) and one return row per routed row of this rank; shapes the
    layer cannot take give 0."""
    from llama_rust_b200.executor import moe_ep_arena_bytes
    n_expert, n_used, n_embd = 8, 2, 4096
    for world in (1, 2, 3, 8):
        e_loc = -(-n_expert // world)
        for t_max in (1, 48, 512):
            n = moe_ep_arena_bytes(n_expert, n_used, n_embd, world, t_max)
            slots = e_loc * world * t_max
            payload = 2 * (slots * (n_embd + 1) * 4 + t_max * n_used * n_embd * 4 + e_loc * world * 4)
            assert payload <= n <= payload + 64 * 256, (world, t_max, n, payload)  # tables start on 256-byte boundaries
            assert n % 256 == 0
        assert moe_ep_arena_bytes(n_expert, n_used, n_embd, world, 64) > moe_ep_arena_bytes(n_expert, n_used, n_embd, world, 32)
    for bad in ((0, 2, 4096, 2, 8), (8, 0, 4096, 2, 8), (8, 9, 4096, 2, 8), (8, 2, 0, 2, 8), (8, 2, 4098, 2, 8), (8, 2, 4096, 0, 8),
                (8, 2, 4096, 9, 8), (8, 2, 4096, 2, 0), (8, 2, 4096, 2, (1 << 20) + 1)):
        with pytest.raises(ValueError):
            moe_ep_arena_bytes(*bad)


def test_header_is_plain_c(tmp_path):
    """The boundary is a C ABI: the header must compile as C99 on its own (what a cgo / bindgen / cbindgen consumer sees)."""
    import shutil
    import subprocess
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    header = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "llama_rust_b200.h")
    src = tmp_path / "use_header.c"
    src.write_text(f'#include "{header}"\nint main(void) {{ llr_exec* e = 0; llr_moe_ep* p = 0; (void)e; (void)p; '
                   'return sizeof(llr_llama_layer) + sizeof(llr_moe_layer) + sizeof(llr_gguf_tensor) > 0 ? 0 : 1; }\n')
    r = subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-pedantic", "-Werror", "-c", str(src), "-o", str(tmp_path / "use_header.o")],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_ctypes_structures_have_the_layout_of_the_header(tmp_path):
    """Every structure that crosses the boundary by value or by pointer: size and the offset of every field as the C
    compiler lays the header's declaration out, against the ctypes mirror the tests and the bench call through."""
    import shutil
    import subprocess
    from llama_rust_b200 import _lib
    gcc = shutil.which("gcc")
    if gcc is None:
        pytest.skip("no C compiler")
    pairs = {"llr_counters": _lib.Counters, "llr_gguf_tensor": _lib.GgufTensor, "llr_program_entry": _lib.ProgramEntry,
             "llr_program_op": _lib.ProgramOp, "llr_program_shard": _lib.ProgramShard, "llr_llama_config": _lib.LlamaConfig,
             "llr_llama_layer": _lib.LlamaLayer, "llr_llama_model": _lib.LlamaModel, "llr_moe_layer": _lib.MoeLayer}
    header = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "llama_rust_b200.h")
    lines = ['#include <stdio.h>', '#include <stddef.h>', f'#include "{header}"', 'int main(void) {']
    for cname, st in pairs.items():
        lines.append(f'  printf("{cname} %zu", sizeof({cname}));')
        for fname, *_ in st._fields_:
            lines.append(f'  printf(" %zu", offsetof({cname}, {fname}));')
        lines.append('  printf("\\n");')
    lines += ['  return 0;', '}']
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines) + "\n")
    exe = tmp_path / "layout"
    r = subprocess.run([gcc, "-std=c99", str(src), "-o", str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr  # a field the mirror names and the header does not fails here
    out = subprocess.run([str(exe)], capture_output=True, text=True, check=True).stdout.split("\n")
    for line in filter(None, out):
        cname, size, *offs = line.split()
        st = pairs[cname]
        assert int(size) == C.sizeof(st), (cname, size, C.sizeof(st))
        assert [int(o) for o in offs] == [getattr(st, f[0]).offset for f in st._fields_], cname
