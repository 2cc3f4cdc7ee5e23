"""The C-ABI shared library loads without a GPU and exports every function include/dist_gnn_b200.h declares."""
import ctypes
import os
import re

from conftest import PKG, ROOT


def declared_functions():
    text = open(os.path.join(ROOT, 'include', 'dist_gnn_b200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return sorted(set(re.findall(r'\b(dg_[a-z0-9_]+)\s*\(', text)))


def test_library_loads_and_exports_every_declared_symbol():
    path = os.path.join(PKG, 'csrc', 'libdist_gnn_b200.so')
    assert os.path.exists(path), 'build the library first: python dist-gnn_b200/csrc/build.py'
    import torch  # noqa: F401  (loads the NCCL the library links against)
    lib = ctypes.CDLL(path)
    names = declared_functions()
    assert len(names) >= 20
    for name in names:
        assert hasattr(lib, name), f'{name} is declared in the header but not exported'
    lib.dg_strerror.restype = ctypes.c_char_p
    assert lib.dg_version() >= 100
    assert lib.dg_strerror(0) == b'ok' and b'row-sorted' in lib.dg_strerror(-3)


def test_argument_checks_need_no_gpu():
    import spmm_cpp
    L = spmm_cpp.lib()
    out = ctypes.c_void_p()
    assert L.dg_plan_create(None, None, -1, 1, 1, None, ctypes.byref(out)) == -2      # negative nnz
    assert L.dg_plan_create(None, None, 5, 1, 1, None, ctypes.byref(out)) == -1       # entries but no arrays
    assert L.dg_plan_create(None, None, 0, 1, 1, None, None) == -1                    # no output slot
    assert L.dg_spmm_csr(None, None, None, 1, None, 1, 1, 1.0, 0.0, 0, None, None, None) == -1
    assert L.dg_comm_create(None, 0, 1, ctypes.byref(out)) == -1
    assert L.dg_plan_destroy(None) == 0 and L.dg_comm_destroy(None) == 0
    # the peer-copy loops and the dense transforms reject missing objects before touching a device
    assert L.dg_comm_peer_alloc(None, 16, None) == -1 and L.dg_comm_peer_open(None, None) == -1 and L.dg_comm_peer_close(None) == -1
    assert L.dg_comm_peer_capacity(None) == 0
    assert L.dg_peer_spmm(None, None, 0, None, None, 0, None, None, None, None, None, 0, 0, None, 0, None) == -1
    assert L.dg_peer_spmm_packed(None, None, 0, None, None, None, 0, None, None, None, None, 0, None, None, None, None, None, 0, 0, None, 0,
                                 None) == -1
    assert L.dg_peer_spmm_packed(None, None, 0, None, None, None, 2, None, None, None, None, 0, None, None, None, None, None, 0, 0, None, 0,
                                 None) == -1                                           # stages without their offsets
    assert L.dg_dense_nt_masked(None, 4, None, None, 4, None, 4, 1, 1, 1, 0, None, 0, None) == -1
    assert L.dg_dense_tn(None, 4, None, 4, None, 4, 1, 1, 1, None, 0, 1, None) == -1
    assert L.dg_dense_supported(0, 1, 1, 4, 4, None, None, None) == 0 and L.dg_dense_tn_supported(1, 300, 1, 300, 4, None, None) == 0


def test_product_modules_do_not_import_the_oracle():
    for folder, _, files in os.walk(PKG):
        for f in files:
            if f.endswith('.py') or f.endswith('.cu') or f.endswith('.h'):
                text = open(os.path.join(folder, f)).read()
                assert not re.search(r'^\s*(from|import)\s+oracle\b|oracle[/.](ref_|spmm_ref|_build|_ref)', text, flags=re.M), \
                    f'{f} reaches into the oracle'


def _top_level_arguments(text, start):
    """Number of arguments of the call whose opening bracket ends at text[start - 1]."""
    depth, commas, empty, i = 1, 0, True, start
    while depth:
        ch = text[i]
        if ch in '([{':
            depth += 1
        elif ch in ')]}':
            depth -= 1
        elif ch == ',' and depth == 1:
            commas += 1
        if depth and not ch.isspace():
            empty = False
        i += 1
    return 0 if empty else commas + 1


def test_c_examples_of_the_integration_guide_match_the_header():
    """Every dg_* call in the guide's C / C++ snippets passes as many arguments as the header's prototype takes."""
    header = open(os.path.join(ROOT, 'include', 'dist_gnn_b200.h')).read()
    header = re.sub(r'//[^\n]*', '', re.sub(r'/\*.*?\*/', '', header, flags=re.S))
    takes = {}
    for m in re.finditer(r'\b(dg_[a-z0-9_]+)\s*\(([^;{]*?)\)\s*;', header, flags=re.S):
        inside = m.group(2).strip()
        takes[m.group(1)] = 0 if inside in ('', 'void') else inside.count(',') + 1
    guide = open(os.path.join(ROOT, 'INTEGRATION.md')).read()
    snippets = re.findall(r'```(?:c|cpp)\n(.*?)```', guide, flags=re.S)
    seen = 0
    for snippet in snippets:
        snippet = re.sub(r'/\*.*?\*/', '', snippet, flags=re.S)
        for m in re.finditer(r'\b(dg_[a-z0-9_]+)\s*\(', snippet):
            assert m.group(1) in takes, f'{m.group(1)} is used in the guide but not declared'
            assert _top_level_arguments(snippet, m.end()) == takes[m.group(1)], f'{m.group(1)}: argument count differs from the header'
            seen += 1
    assert seen >= 15
