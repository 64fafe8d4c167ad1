"""Prints the lines to add to ferro_b200/csrc/chain_programs.def for a chain.

The library compiles the chains listed in that manifest ahead of time; any
other chain runs on the interpreter.  Write the chain with the host-side
helpers, say which operands are contiguous / broadcast / transposed, and paste
the output into the manifest:

    from ferro_b200.backend import BinaryKind as B, ChainStep as S, UnaryKind as U, T
    from ferro_b200.chain_manifest import manifest_lines
    print(manifest_lines("ProgSwish", [S.Load(0), S.Unary(U.Sigmoid), S.Binary(B.Mul, other=0)],
                         tile_classes=[("staged",)]))

then rebuild with `python -m ferro_b200.build`.
"""
from typing import Optional, Sequence

from . import kinds as K

_UN = {getattr(K, n): "FB_" + n for n in dir(K) if n.startswith("UN_")}
_BIN = {getattr(K, n): "FB_" + n for n in dir(K) if n.startswith("BIN_")}
_CLASS = {"direct": "kOpDirect", "bcast": "kOpBcastB", "staged": "kOpStaged"}
# FB_UN_POWF / FB_UN_CLAMP are resolved on the host before a call is matched (math.cuh).
_POWF = {0.5: "FBI_POWF_SQRT", -0.5: "FBI_POWF_RSQRT", -1.0: "FBI_POWF_RCP", -2.0: "FBI_POWF_RSQ",
         2.0: "FBI_POWF_SQ", 3.0: "FBI_POWF_CUBE", 1.5: "FBI_POWF_1_5"}


def _unary(step):
    if step.kind == K.UN_POWF:
        return _POWF.get(float(step.p0), "FBI_POWF_GENERIC")
    if step.kind == K.UN_CLAMP:
        return "FBI_CLAMP_ORDERED"  # bounds that are not NaN; a NaN bound keeps FB_UN_CLAMP
    return _UN[step.kind]


def manifest_lines(name: str, steps: Sequence, seg: bool = True,
                   tile_classes: Optional[Sequence[Sequence[str]]] = None, comment: str = "") -> str:
    """`steps`: ChainStep list.  `seg`: compile for contiguous / broadcast operands.  `tile_classes`: one
    tuple per tile instantiation giving each operand's class, "direct" | "bcast" | "staged"."""
    parts = []
    for s in steps:
        r = "V" if s.dst == 0 else "T"
        if s.opcode == 0:
            parts.append(f"Load{r}({s.src})")
        elif s.opcode == 1:
            parts.append(f"Un{r}({_unary(s)})")
        elif s.opcode == 2:
            if s.src & 64:
                raise ValueError("swapped binary steps have no manifest helper yet: write SS{...} by hand")
            src = s.src & ~64
            where = "kOther" if src == 0 else "kImm" if src == 1 else f"Op({src - 8})"
            parts.append(f"Bin{r}({_BIN[s.kind]}, {where})")
        else:
            raise ValueError("immediate loads are written by hand: SS{FB_CH_IMM, dst, 0, 0, 0}")
    out = []
    if comment:
        out.append(f"// {comment}")
    out.append(f"FB_CHAIN_PROGRAM({name}, " + ", ".join(parts) + ")")
    if seg:
        out.append(f"FB_CHAIN_SEG({name})")
    for cls in tile_classes or []:
        c = [_CLASS[x] for x in cls] + ["kOpDirect"] * (3 - len(cls))
        out.append(f"FB_CHAIN_TILE({name}, {', '.join(c[:3])})")
    return "\n".join(out)


if __name__ == "__main__":
    from .backend import BinaryKind as B, ChainStep as S, T, UnaryKind as U
    demo = [S.Load(0), S.Unary(U.Abs), S.Unary(U.Neg), S.Unary(U.Exp), S.Load(1, dst=T), S.Unary(U.Abs, dst=T),
            S.Binary(B.Add, imm=1.0, dst=T), S.Unary(U.Sqrt, dst=T), S.Binary(B.Mul), S.Unary(U.Tanh), S.Load(2, dst=T),
            S.Unary(U.Powf(1.5), dst=T), S.Binary(B.Add), S.Unary(U.Clamp(-1.0, 1.0))]
    print(manifest_lines("ProgGateClamp", demo, tile_classes=[("direct", "bcast", "staged")],
                         comment="clamp(tanh(exp(-abs(x0)) * sqrt(abs(x1) + c)) + powf(x2, 1.5), lo, hi)"))
