"""Shared helpers for the parity tests."""
import numpy as np


def qp_of(oracle, row):
    return oracle.qp(np.float32(row[0]), int(row[1]))


def ltq_qp(row):
    import ltq
    return ltq.QParams(float(np.float32(row[0])), int(row[1]))


def iter_qmm_cases(g):
    n = int(g["count"][0])
    for i in range(n):
        key = f"c{i}"
        if key + ".meta" not in g:
            continue
        M, N, K, tA, tB, use_bias, qi = [int(v) for v in g[key + ".meta"]]
        yield dict(key=key, M=M, N=N, K=K, tA=tA, tB=tB, qp=g[key + ".qp"], A=g[key + ".A"], B=g[key + ".B"],
                   bias=g[key + ".bias"] if use_bias else None, C=g[key + ".C"], ws=g[key + ".ws"])


def iter_conv_cases(g):
    for i, row in enumerate(g["cases"]):
        B, Cin, H, W, Cout, kh, kw, ph, pw, sh, sw, use_bias = [int(v) for v in row]
        key = f"v{i}"
        yield dict(key=key, B=B, Cin=Cin, H=H, W=W, Cout=Cout, kh=kh, kw=kw, ph=ph, pw=pw, sh=sh, sw=sw, qp=g[key + ".qp"],
                   x=g[key + ".x"], w=g[key + ".w"], bias=g[key + ".bias"] if use_bias else None, y=g[key + ".y"],
                   col0=g[key + ".col0"])
