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
