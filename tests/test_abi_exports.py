"""CPU: the C-ABI library loads without a GPU and exports exactly the entry points include/b200_moe.h declares;
the ctypes table and the ctypes mirror of B200MoeBlock agree with the header. No kernel is launched."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "b200_moe.h")


def declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)  # comments mention entry points too
    return sorted(set(re.findall(r"\b(b200_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_entry_point():
    from ml_dataflow_b200 import _lib, build

    build.build()
    lib = ctypes.CDLL(_lib.LIB_PATH)
    names = declared_functions()
    assert len(names) >= 30
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in include/b200_moe.h but not exported"
    # the Python binding table covers the same set, no more and no less
    assert sorted(_lib.SIGNATURES) == names
    assert _lib.load() is not None


def test_argument_counts_match_the_header():
    from ml_dataflow_b200 import _lib

    text = re.sub(r"/\*.*?\*/", "", open(HEADER).read(), flags=re.S)
    for name, (_, argtypes) in _lib.SIGNATURES.items():
        m = re.search(r"\b" + name + r"\s*\(([^)]*)\)\s*;", text, flags=re.S)
        assert m, name
        args = m.group(1).strip()
        n = 0 if args in ("", "void") else len(args.split(","))
        assert n == len(argtypes), f"{name}: header has {n} parameters, ctypes table {len(argtypes)}"


def test_block_structure_mirror_matches_the_header():
    from ml_dataflow_b200 import _lib

    text = open(HEADER).read()
    body = re.search(r"typedef struct B200MoeBlock \{(.*?)\} B200MoeBlock;", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        for part in decl.split(","):
            fields.append(re.findall(r"[A-Za-z_][A-Za-z0-9_]*", part)[-1])
    assert fields == [f[0] for f in _lib.MoeBlock._fields_]
    # 5 ints (+4 pad), then only 8-byte members
    assert ctypes.sizeof(_lib.MoeBlock) == 24 + 8 * (len(fields) - 5)


def test_host_only_entry_points_answer_without_a_gpu():
    """Sizing functions run on the host: scratch for the mapping grows with the problem and stays 16-byte granular;
    the built-in scratch of the no-allocation variant is 4 MiB and holds the benchmark's shapes."""
    from ml_dataflow_b200 import _lib

    lib = _lib.load()
    ws = lib.b200_build_expert_mapping_workspace_bytes
    cap = lib.b200_build_expert_mapping_static_capacity_bytes()
    assert cap == 4 << 20
    prev = 0
    for T in (1, 1000, 8192, 32768, 65536, 1 << 20):
        n = ws(T, 64, 8)
        assert n >= prev and n > 0 and n % 4 == 0
        prev = n
        assert n <= cap                      # 64 experts fit the built-in scratch at any token count
    assert ws(1 << 20, 4096, 8) > cap        # a problem the no-allocation variant must refuse
    assert ws(8192, 64, 8) <= ws(8192, 256, 8)


def _struct_fields(name):
    text = open(HEADER).read()
    body = re.search(r"typedef struct " + name + r" \{(.*?)\} " + name + ";", text, flags=re.S).group(1)
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        for part in decl.split(","):
            fields.append(re.findall(r"[A-Za-z_][A-Za-z0-9_]*", part)[-1])
    return fields


def test_transformer_block_structure_mirrors_match_the_header():
    from ml_dataflow_b200 import _lib

    for name, mirror in (("B200TransformerBlock", _lib.TransformerBlock), ("B200TransformerBlockGrads", _lib.TransformerBlockGrads),
                         ("B200TransformerBlockScratch", _lib.TransformerBlockScratch)):
        assert _struct_fields(name) == [f[0] for f in mirror._fields_], name
    # the MoE part sits inside the block structure by value
    assert dict(_lib.TransformerBlock._fields_)["moe"] is _lib.MoeBlock


def test_attention_workspace_sizes_and_argument_checks_without_a_gpu():
    """Host-side logic only: the workspace formula and the argument checks run before any CUDA call."""
    from ml_dataflow_b200 import _lib

    lib = _lib.load()
    ws = lib.b200_attention_workspace_bytes
    up = lambda v: (v + 255) // 256 * 256
    T, Hq, Hkv = 1000, 16, 4
    # head size 128: fused both ways - nothing for inference, the fp32 dQ accumulator and delta for training
    assert ws(0, Hq, Hkv, 128, T, 600, 600) == 0
    assert ws(1, Hq, Hkv, 128, T, 600, 600) == up(T * Hq * 128 * 4) + up(T * Hq * 4)
    # head size 64: fused forward, GEMM-by-GEMM backward (score matrices of one head and query chunk)
    assert ws(0, Hq, Hkv, 64, T, 600, 600) == 0
    assert ws(1, Hq, Hkv, 64, T, 600, 600) >= 600 * 600 * 6
    # other head sizes: GEMM by GEMM both ways
    assert ws(0, Hq, Hkv, 32, T, 600, 600) >= 600 * 600 * 6
    assert ws(1, 0, Hkv, 128, T, 600, 600) == 0  # nonsense in, 0 out
    # query heads must be a multiple of the key/value heads; only bf16; lengths within the stated maxima
    ia = lambda *v: (ctypes.c_int * len(v))(*v)
    bad = lib.b200_attention_fwd(5, 1, 8, 8, ia(0), ia(8), 8, ia(0), ia(8), 8, 3, 2, 128, None, None, None, None, None, 1, 0, None, None)
    assert bad == -1
    assert lib.b200_attention_fwd(3, 1, 8, 8, ia(0), ia(8), 8, ia(0), ia(8), 8, 4, 2, 128, None, None, None, None, None, 1, 0, None, None) == -1
    assert lib.b200_attention_fwd(5, 1, 8, 8, ia(0), ia(9), 8, ia(0), ia(9), 8, 4, 2, 128, None, None, None, None, None, 1, 0, None, None) == -1


def test_block_driver_refuses_bad_arguments_without_a_gpu():
    """The block driver checks its structure before any CUDA call: null block, inconsistent MoE part."""
    from ml_dataflow_b200 import _lib

    lib = _lib.load()
    assert lib.b200_transformer_block_fwd(None, None, None, None) == -1
    blk = _lib.TransformerBlock()  # all zeros: bad dimensions
    assert lib.b200_transformer_block_fwd(ctypes.byref(blk), None, None, None) == -1
    assert lib.b200_transformer_block_bwd(ctypes.byref(blk), None, None, None, None, None) == -1
