"""K-chunk decayed terms that the reference's pairwise executor runs (tests/test_decayed_lower.py:
440-482 there) and that are NOT decayed attention of one sequence at one rate: a decay-row gate on
the intra-chunk element, another rate in the intra masks of the later arms, a cross pair left out.
Test helper: builds catopt IR, so it needs catopt importable."""
from __future__ import annotations


def variant_term(B: int, H: int, T: int, d: int, C: int, scale: float, *, intra_row: bool = False,
                 second_rate: bool = False, drop_pair: bool = False, gate_inside: bool = False):
    from catopt_core.ir import IR, Const, Op, Param, TensorType, Var

    K = T // C
    tt = lambda *s: TensorType(tuple(s))  # noqa: E731
    q, k, v = (Var(n, tt(B, H, T, d)) for n in "qkv")
    g, g2 = Param("g", tt(H)), Param("g2", tt(H))
    sc = Const(scale)
    sizes = [C] * K
    rows = lambda t, i: Op.make("split", t, dim=-2, index=i, sizes=sizes)  # noqa: E731
    kt = Op.make("transpose", k, dim0=-1, dim1=-2)
    cols = lambda i: Op.make("split", kt, dim=-1, index=i, sizes=sizes)  # noqa: E731
    vec = lambda **kw: Op.make("unsqueeze", Op.make("decay_vec", g, t=C, **kw), dim=-1)  # noqa: E731

    def pair(i, j):
        keys = Op.make("transpose", Op.make("mul", rows(k, j), vec(sign=-1, offset=0)), dim0=-1, dim1=-2)
        body = Op.make("matmul", rows(q, i), Op.make("matmul", keys, rows(v, j)))
        gate = vec(sign=1, offset=(i - j) * C)
        if gate_inside:
            return Op.make("div", Op.make("mul", gate, body), sc)
        return Op.make("mul", gate, Op.make("div", body, sc))

    def arm(i):
        rate = g2 if (second_rate and i > 0) else g
        t = Op.make("div", Op.make("om_decayed", Op.make("matmul", rows(q, i), cols(i)),
                                   Op.make("decay", rate, t=C), rows(v, i)), sc)
        if intra_row:
            t = Op.make("mul", vec(sign=1, offset=C), t)
        for j in range(i):
            if drop_pair and i == K - 1 and j == 0:
                continue
            t = Op.make("add", t, pair(i, j))
        return t

    params = {"g": g, "g2": g2} if second_rate else {"g": g}
    return IR(root=Op.make("concat", *[arm(i) for i in range(K)], dim=-2), inputs=[q, k, v],
              input_names={"q", "k", "v"}, params=params)
