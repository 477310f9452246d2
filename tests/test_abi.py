"""CPU checks of the boundary: the shared library builds, loads and exports every symbol
the headers declare; the host facade validates graphs; nothing computes without a GPU."""
import ctypes as C
import os
import re

import numpy as np
import pytest

import util
from cnet_b200 import configs, lib as cl
from cnet_b200.net import Net

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared(header):
    txt = open(os.path.join(ROOT, "include", header)).read()
    txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
    return sorted(set(re.findall(r"\b(cn[bh]_[a-z0-9_]+)\s*\(", txt)))


def test_library_exports_every_declared_symbol(built_lib):
    lib = C.CDLL(built_lib)
    names = _declared("cnet_b200.h") + _declared("cnet_b200_host.h")
    assert len(names) > 50
    for n in names:
        assert hasattr(lib, n), "missing export " + n
        assert n in cl.SIGNATURES or n in ("cnh_bucket_hook",), "no ctypes signature for " + n


def test_python_binding_covers_headers(built_lib):
    declared = set(_declared("cnet_b200.h") + _declared("cnet_b200_host.h")) - {"cnh_bucket_hook"}
    assert declared == set(cl.SIGNATURES)


def test_no_gpu_means_loud_failure(built_lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    net = Net()
    configs.build_classifier(net, n=16, m=4)
    with pytest.raises(cl.CnetError):
        net.allocate(2)
    # the raw C ABI refuses too: no device, no context
    lib = cl.load()
    ctx = C.c_void_p()
    assert lib.cnb_create(0, 1 << 20, C.byref(ctx)) < 0
    assert lib.cnb_last_error()


def test_forward_before_allocate_is_an_error(built_lib):
    net = Net()
    configs.build_classifier(net, n=16, m=4)
    with pytest.raises(cl.CnetError, match="allocateOnGpu"):
        net.forward()


def test_graph_validation(built_lib):
    net = Net()
    x = net.add(configs.INPUT, 8)
    with pytest.raises(cl.CnetError):
        net.add(configs.GELU, 8, prev=[x + 5])          # unknown producer
    net2 = Net()
    a = net2.add(configs.INPUT, 8)
    with pytest.raises(cl.CnetError):
        net2.add(configs.GELU, 4, prev=[a])             # producer larger than the input block
    lib = cl.load()
    assert lib.cnh_add(net2.h, configs.LINEAR, 3, 10, 0, None, 0) < 0   # in2 not a multiple of in1
    assert lib.cnh_add(net2.h, 99, 1, 0, 0, None, 0) < 0                # unknown type id


def test_out_sizes_follow_reference_constructors(built_lib):
    net = Net()
    spec = configs.build_embed_lm(net, tokens=4, vocab=32, dim=8, hidden=16)
    L = spec.layers
    assert net.out_size(L["emb"]) == 32           # max tokens * dim (impl/embed.h:43-47)
    assert net.out_size(L["l1"]) == 16            # in2 / in1 (impl/linear.h:18-23)
    assert net.out_size(L["sm"]) == 32
    assert net.out_size(L["ce"]) == 1             # impl/crossent.h:14-17


def test_case_inputs_are_deterministic():
    a = util.case_inputs("embed_lm_small")
    b = util.case_inputs("embed_lm_small")
    assert np.array_equal(a[2][0][0], b[2][0][0])
    assert a[2][0][0][0, -1] == -1


def test_reference_style_user_layer_compiles_and_is_refused(built_lib, tmp_path):
    """tests/cpp/user_layer_probe.cpp: a layer with the reference's dz / dz_star contract compiles against
    the facade header; CNet::add refuses it with a message unless it runs its own device kernels."""
    import subprocess
    here = os.path.dirname(os.path.abspath(__file__))
    exe = str(tmp_path / "probe")
    libdir = os.path.dirname(built_lib)
    env = dict(os.environ)
    env.pop("CXX", None)
    subprocess.run(["g++", "-std=c++17", "-I/usr/local/cuda/include", os.path.join(here, "cpp", "user_layer_probe.cpp"),
                    "-o", exe, "-L" + libdir, "-l:libcnet_b200.so", "-Wl,-rpath," + libdir], check=True, env=env)
    r = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    assert r.returncode == 0 and "OK" in r.stdout, r.stdout


def test_struct_layouts_of_the_python_binding_match_the_header(tmp_path):
    """cnb_split_span is passed by pointer through ctypes: size and field offsets of the Python mirror must be
    what a C compiler makes of include/cnet_b200.h."""
    import ctypes as C
    import subprocess
    from cnet_b200 import lib as L
    here = os.path.dirname(os.path.abspath(__file__))
    src = tmp_path / "layout.c"
    src.write_text(
        '#include <stdio.h>\n#include <stddef.h>\n#include "cnet_b200.h"\n'
        'int main(void) {\n'
        '  printf("%zu %zu %zu %zu %zu %zu\\n", sizeof(cnb_split_span), offsetof(cnb_split_span, begin), offsetof(cnb_split_span, count),\n'
        '         offsetof(cnb_split_span, hi), offsetof(cnb_split_span, h16), offsetof(cnb_split_span, l16));\n'
        '  return 0;\n}\n')
    exe = str(tmp_path / "layout")
    subprocess.run(["gcc", "-I", os.path.join(here, "..", "include"), "-I/usr/local/cuda/include", str(src), "-o", exe], check=True)
    out = subprocess.run([exe], stdout=subprocess.PIPE, text=True, check=True).stdout.split()
    S = L.SplitSpan
    want = [C.sizeof(S), S.begin.offset, S.count.offset, S.hi.offset, S.h16.offset, S.l16.offset]
    assert [int(v) for v in out] == want
