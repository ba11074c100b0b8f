"""ctypes face of the fp64 oracle (``csrc/ref/refmodel.cc``): the CPU double-precision decoder that
device results are checked against. Supports what the reference's oracle supports (MHA, learned
positions, tied head) plus GQA, RoPE, N(0, std) initialisation and a mixture-of-experts MLP (softmax
router, top-k, renormalised weights)."""
from __future__ import annotations

import ctypes
from ctypes import POINTER, c_char_p, c_double, c_int, c_longlong, c_size_t, c_uint64, c_void_p

import numpy as np

from .. import plan as planlib


def _lib():
    L = planlib.lib()
    if not getattr(L, "_cai_ref_declared", False):
        L.cai_ref_create.argtypes = [c_int] * 8 + [c_double, c_int, c_double, c_int, c_double, c_uint64]
        L.cai_ref_create.restype = c_void_p
        L.cai_ref_create_moe.argtypes = [c_int] * 8 + [c_double, c_int, c_double, c_int, c_double, c_int, c_int, c_uint64]
        L.cai_ref_create_moe.restype = c_void_p
        L.cai_ref_free.argtypes = [c_void_p]
        L.cai_ref_free.restype = None
        L.cai_ref_param_count.argtypes = [c_void_p]
        L.cai_ref_param_count.restype = c_size_t
        for fn in ("cai_ref_params", "cai_ref_grads"):
            getattr(L, fn).argtypes = [c_void_p]
            getattr(L, fn).restype = POINTER(c_double)
        L.cai_ref_offset.argtypes = [c_void_p, c_char_p, POINTER(c_size_t)]
        L.cai_ref_offset.restype = c_longlong
        L.cai_ref_forward.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
        L.cai_ref_forward.restype = c_double
        L.cai_ref_backward.argtypes = [c_void_p, c_int, c_void_p, c_void_p]
        L.cai_ref_backward.restype = None
        L.cai_ref_adamw.argtypes = [c_void_p, c_double, c_double, c_double, c_double, c_double]
        L.cai_ref_adamw.restype = None
        L.cai_ref_accuracy.argtypes = [c_void_p, c_int, c_void_p]
        L.cai_ref_accuracy.restype = c_double
        L.cai_ref_grad_check.argtypes = [c_void_p, c_int, c_void_p, c_void_p, c_int, c_double]
        L.cai_ref_grad_check.restype = c_double
        L._cai_ref_declared = True
    return L


class Oracle:
    def __init__(self, vocab=64, seq=32, hidden=64, layers=2, n_heads=4, n_kv_heads=None, head_dim=16, ffn=128,
                 eps=1e-6, rope=False, rope_theta=10000.0, tied=True, init_std=0.0, seed=1, experts=0, top_k=2):
        self.L = _lib()
        self.seq, self.vocab = seq, vocab
        if experts:
            self.h = self.L.cai_ref_create_moe(vocab, seq, hidden, layers, n_heads, n_kv_heads or n_heads, head_dim, ffn,
                                               eps, int(rope), rope_theta, int(tied), init_std, experts, top_k, seed)
        else:
            self.h = self.L.cai_ref_create(vocab, seq, hidden, layers, n_heads, n_kv_heads or n_heads, head_dim, ffn, eps,
                                           int(rope), rope_theta, int(tied), init_std, seed)
        if not self.h:
            raise ValueError("invalid oracle spec")
        n = self.L.cai_ref_param_count(self.h)
        self.params = np.ctypeslib.as_array(self.L.cai_ref_params(self.h), shape=(n,))
        self.grads = np.ctypeslib.as_array(self.L.cai_ref_grads(self.h), shape=(n,))

    @staticmethod
    def _i32(a):
        return np.ascontiguousarray(np.asarray(a, dtype=np.int32).reshape(-1))

    def tensor(self, name, grad=False):
        cnt = c_size_t(0)
        off = self.L.cai_ref_offset(self.h, name.encode(), ctypes.byref(cnt))
        if off < 0:
            raise KeyError(name)
        return (self.grads if grad else self.params)[off:off + cnt.value]

    def forward(self, tokens, targets):
        t, y = self._i32(tokens), self._i32(targets)
        return self.L.cai_ref_forward(self.h, t.size // self.seq, t.ctypes.data, y.ctypes.data)

    def backward(self, tokens, targets):
        t, y = self._i32(tokens), self._i32(targets)
        self.L.cai_ref_backward(self.h, t.size // self.seq, t.ctypes.data, y.ctypes.data)

    def adamw(self, lr, b1=0.9, b2=0.999, eps=1e-8, wd=0.01):
        self.L.cai_ref_adamw(self.h, lr, b1, b2, eps, wd)

    def accuracy(self, targets):
        y = self._i32(targets)
        return self.L.cai_ref_accuracy(self.h, y.size // self.seq, y.ctypes.data)

    def grad_check(self, tokens, targets, n_probe=0, h=1e-5):
        t, y = self._i32(tokens), self._i32(targets)
        return self.L.cai_ref_grad_check(self.h, t.size // self.seq, t.ctypes.data, y.ctypes.data, n_probe, h)

    def close(self):
        if self.h:
            self.L.cai_ref_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def load_engine_weights(oracle: Oracle, engine):
    """Copy an engine's (tp = 1) parameters into an oracle of the same architecture. The engine
    stores weights as [out, in]; the oracle applies Y = X W with W stored [in, out]."""
    m = engine.model
    hq, hkv = m.num_heads * m.head_dim, m.num_kv_heads * m.head_dim

    def put(name, value):
        oracle.tensor(name)[:] = value.double().cpu().numpy().reshape(-1)

    put("E", engine.param("embed"))
    put("gf", engine.param("gf"))
    if "lm_head" in engine.named:
        put("head", engine.param("lm_head"))
    for l in range(m.num_layers):
        wqkv = engine.param(f"L{l}.wqkv").float()
        put(f"L{l}.g1", engine.param(f"L{l}.g1"))
        put(f"L{l}.Wq", wqkv[:hq].t().contiguous())
        put(f"L{l}.Wk", wqkv[hq:hq + hkv].t().contiguous())
        put(f"L{l}.Wv", wqkv[hq + hkv:].t().contiguous())
        put(f"L{l}.Wo", engine.param(f"L{l}.wo").float().t().contiguous())
        put(f"L{l}.g2", engine.param(f"L{l}.g2"))
        wgu = engine.param(f"L{l}.wgu").float()
        f = m.ffn_hidden
        put(f"L{l}.Wg", wgu[:f].t().contiguous())
        put(f"L{l}.Wu", wgu[f:].t().contiguous())
        put(f"L{l}.Wd", engine.param(f"L{l}.wd").float().t().contiguous())
