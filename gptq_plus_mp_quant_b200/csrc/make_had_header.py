"""Writes ``rq_had_tables.cuh``: the 12 x 12, 20 x 20 and 28 x 28 Hadamard matrices that ``get_hadK`` hands out, as
compile-time sign tables for the rotation kernel's fixed-matrix mix.

    python -m gptq_plus_mp_quant_b200.csrc.make_had_header
"""
from __future__ import annotations

import os

from ..utils.hadamard_utils import hadamard_of_order

HERE = os.path.dirname(os.path.abspath(__file__))


def main() -> None:
    lines = ["// Sign tables of the K x K Hadamard matrices of orders 12, 20 and 28 (written by make_had_header.py; do not",
             "// edit): bit c of had_row<K>(r) is set where entry (r, c) is +1.", "#pragma once", "",
             "#include <stdint.h>", "", "namespace rq {", "namespace fwht {", "",
             "template <int K> __host__ __device__ constexpr uint32_t had_row(int r);"]
    for K in (12, 20, 28):
        H = hadamard_of_order(K)
        rows = []
        for r in range(K):
            bits = 0
            for c in range(K):
                if H[r, c] > 0:
                    bits |= 1 << c
            rows.append(f"0x{bits:08x}u")
        lines.append(f"template <> __host__ __device__ constexpr uint32_t had_row<{K}>(int r) {{")
        lines.append(f"    constexpr uint32_t t[{K}] = {{")
        for i in range(0, K, 6):
            lines.append("        " + ", ".join(rows[i:i + 6]) + ",")
        lines.append("    };")
        lines.append("    return t[r];")
        lines.append("}")
    lines += ["", "}  // namespace fwht", "}  // namespace rq", ""]
    with open(os.path.join(HERE, "rq_had_tables.cuh"), "w") as f:
        f.write("\n".join(lines))


if __name__ == "__main__":
    main()
