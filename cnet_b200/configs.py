"""The benchmark nets (as layer lists) and their seeded synthetic inputs.

A *builder* takes any object with the flat net interface
``add(type, a, b, c, prev) -> uid`` (the device net, or a CPU checker in the tests) and
adds the layers in an order in which every producer precedes its consumers, as the
reference's insertion-ordered forward requires (impl/cnet.h:366-377).  It returns a
``NetSpec`` naming the data input, the loss, and every weight with its init variance.

Synthetic data stands in for MNIST / text (not available offline): shapes, value ranges
and distributions follow the benchmark configurations.
"""
from dataclasses import dataclass, field

import numpy as np

# layer type ids: the reference's own (impl/cnet.h:31-44)
HADAMARD, EMBEDDING, LINEAR, FOURIER, CROSSENT, RESIDUAL, SOFTMAX, INPUT, CRELU, GELU, L2OUT, TRIFOURIER = range(1, 13)


@dataclass
class NetSpec:
    name: str
    main: int                      # uid of the data CInput / CEmbedding
    loss: int                      # uid of the CrossEntropy
    in_dim: int                    # complex elements (or tokens) per sample
    n_classes: int
    weights: list = field(default_factory=list)    # [(uid, length, std)]
    tokens: bool = False
    vocab: int = 0
    layers: dict = field(default_factory=dict)     # name -> uid


def build_classifier(net, n=784, m=10):
    """Config 1: CInput(n) -> FourierTrans -> Hadamard(h) -> CGelu -> Linear(n->m) -> CrossEntropy."""
    x = net.add(INPUT, n)
    ft = net.add(FOURIER, n, prev=[x])
    h = net.add(INPUT, n)
    had = net.add(HADAMARD, n, prev=[ft, h])
    g = net.add(GELU, n, prev=[had])
    w = net.add(INPUT, n * m)
    lin = net.add(LINEAR, n, n * m, prev=[g, w])
    ce = net.add(CROSSENT, m, prev=[lin])
    s = n ** -0.5
    return NetSpec("classifier", x, ce, n, m, [(h, n, s), (w, n * m, s)],
                   layers=dict(x=x, ft=ft, h=h, had=had, gelu=g, w=w, lin=lin, ce=ce))


def build_linear(net, n_in=4096, n_out=4096, m=None):
    """Config 2 as a net: CInput(n_in) -> Linear(n_in->n_out) -> CrossEntropy(n_out)."""
    x = net.add(INPUT, n_in)
    w = net.add(INPUT, n_in * n_out)
    lin = net.add(LINEAR, n_in, n_in * n_out, prev=[x, w])
    ce = net.add(CROSSENT, n_out, prev=[lin])
    return NetSpec("linear", x, ce, n_in, n_out, [(w, n_in * n_out, n_in ** -0.5)],
                   layers=dict(x=x, w=w, lin=lin, ce=ce))


def build_mixer(net, n=1024, blocks=8, m=10):
    """Config 3: blocks x [FourierTrans -> Hadamard(h) -> CGelu -> Linear(n->n) -> Residual] -> Linear(n->m) -> CE."""
    x = net.add(INPUT, n)
    s = n ** -0.5
    weights, layers = [], dict(x=x)
    cur = x
    for b in range(blocks):
        ft = net.add(FOURIER, n, prev=[cur])
        h = net.add(INPUT, n)
        had = net.add(HADAMARD, n, prev=[ft, h])
        g = net.add(GELU, n, prev=[had])
        w = net.add(INPUT, n * n)
        lin = net.add(LINEAR, n, n * n, prev=[g, w])
        res = net.add(RESIDUAL, n, prev=[lin, cur])
        weights += [(h, n, s), (w, n * n, s)]
        layers.update({"ft%d" % b: ft, "h%d" % b: h, "had%d" % b: had, "gelu%d" % b: g,
                       "w%d" % b: w, "lin%d" % b: lin, "res%d" % b: res})
        cur = res
    wh = net.add(INPUT, n * m)
    head = net.add(LINEAR, n, n * m, prev=[cur, wh])
    ce = net.add(CROSSENT, m, prev=[head])
    weights.append((wh, n * m, s))
    layers.update(wh=wh, head=head, ce=ce)
    return NetSpec("mixer", x, ce, n, m, weights, layers=layers)


def build_embed_lm(net, tokens=64, vocab=8192, dim=256, hidden=2048):
    """Config 4: CEmbedding(dim, tokens, vocab) -> Linear -> CGelu -> Linear(->vocab) -> SoftMax -> CrossEntropy."""
    emb = net.add(EMBEDDING, dim, tokens, vocab)
    d = tokens * dim
    w1 = net.add(INPUT, d * hidden)
    l1 = net.add(LINEAR, d, d * hidden, prev=[emb, w1])
    g = net.add(GELU, hidden, prev=[l1])
    w2 = net.add(INPUT, hidden * vocab)
    l2 = net.add(LINEAR, hidden, hidden * vocab, prev=[g, w2])
    sm = net.add(SOFTMAX, vocab, prev=[l2])
    ce = net.add(CROSSENT, vocab, prev=[sm])
    # table std 0.02 (N(0, 0.02) read as a standard deviation, the usual LM embedding init)
    return NetSpec("embed_lm", emb, ce, tokens, vocab,
                   [(emb, vocab * dim, 0.02), (w1, d * hidden, d ** -0.5), (w2, hidden * vocab, hidden ** -0.5)],
                   tokens=True, vocab=vocab,
                   layers=dict(emb=emb, w1=w1, l1=l1, gelu=g, w2=w2, l2=l2, sm=sm, ce=ce))


def build_relu_tri(net, n=24, m=6):
    """The layers no benchmark config uses: CInput -> TriangFourier -> CRelu -> Linear(n->m) -> L2Out."""
    x = net.add(INPUT, n)
    tf = net.add(TRIFOURIER, n, prev=[x])
    r = net.add(CRELU, n, prev=[tf])
    w = net.add(INPUT, n * m)
    lin = net.add(LINEAR, n, n * m, prev=[r, w])
    out = net.add(L2OUT, m, prev=[lin])
    return NetSpec("relu_tri", x, out, n, m, [(w, n * m, n ** -0.5)],
                   layers=dict(x=x, tf=tf, relu=r, w=w, lin=lin, ce=out))


def _rng(seed, stream):
    return np.random.Generator(np.random.Philox(key=[int(seed), int(stream)]))


def init_weights(spec, seed=0):
    """{uid: (re, im)} fp32 planes, real and imag parts iid N(0, std^2); one stream per weight."""
    out = {}
    for k, (uid, n, std) in enumerate(spec.weights):
        r = _rng(seed, 1000 + k)
        out[uid] = ((r.standard_normal(n) * std).astype(np.float32),
                    (r.standard_normal(n) * std).astype(np.float32))
    return out


def make_batch(spec, batch, seed=0, step=0, kind=None):
    """Seeded synthetic batch: (x_re, x_im) or tokens, and labels.

    kind "image": real parts uniform [0,1), imag 0 (config 1); "normal": real and imag
    N(0,1) (config 3); for token nets ids uniform over the vocab.
    """
    r = _rng(seed, 10_000_000 + step)
    labels = r.integers(0, spec.n_classes, batch).astype(np.int32)
    if spec.tokens:
        tok = r.integers(0, spec.vocab, (batch, spec.in_dim)).astype(np.int32)
        return tok, labels
    if kind is None:
        kind = "image" if spec.name == "classifier" else "normal"
    if kind == "image":
        xr = r.random((batch, spec.in_dim), dtype=np.float32)
        xi = np.zeros((batch, spec.in_dim), np.float32)
    elif kind == "normal":
        xr = r.standard_normal((batch, spec.in_dim)).astype(np.float32)
        xi = r.standard_normal((batch, spec.in_dim)).astype(np.float32)
    else:  # "fanin": N(0, 1/in_dim) (config 2 inputs)
        s = spec.in_dim ** -0.5
        xr = (r.standard_normal((batch, spec.in_dim)) * s).astype(np.float32)
        xi = (r.standard_normal((batch, spec.in_dim)) * s).astype(np.float32)
    return (xr, xi), labels
