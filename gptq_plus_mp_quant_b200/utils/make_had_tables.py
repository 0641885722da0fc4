"""Writes ``_had_tables.py``: the K x K (+-1) Hadamard matrices of the orders that have no Paley construction here
(52, 92, 100, 116, 124, 156, 172, 188, 212, 228, 236, 244, 252), bit-packed, taken from the reference project's
``utils/had_mat.pt`` so that ``get_hadK`` returns the same matrix for every width the reference supports (e.g.
11008 = 172 * 64).

    python -m gptq_plus_mp_quant_b200.utils.make_had_tables /path/to/reference/utils/had_mat.pt

Each matrix is stored row-major, one bit per entry (1 = +1), base64 over 76-column lines.  The digests of the
matrices are checked by tests/test_hadamard_tables.py against those recorded when the golden fixtures were made.
"""
from __future__ import annotations

import base64
import os
import sys

import numpy as np
import torch

from .hadamard_utils import TABLE_ORDERS, _PALEY2_ORDERS, _is_prime


def generated(K: int) -> bool:
    return K in _PALEY2_ORDERS or (_is_prime(K - 1) and (K - 1) % 4 == 3 and K not in (212, 228, 252))


def main(path: str) -> None:
    table = torch.load(path)
    lines = ['"""Bit-packed Hadamard matrices of the orders without a Paley construction (written by make_had_tables.py;',
             'do not edit).  PACKED[K] = base64 of the row-major K*K bits, 1 = +1, 0 = -1."""', "", "PACKED = {"]
    for K in TABLE_ORDERS:
        if generated(K):
            continue
        m = table[K].to(torch.int8).numpy()
        assert m.shape == (K, K) and set(np.unique(m)) <= {-1, 1}
        bits = np.packbits((m.reshape(-1) > 0).astype(np.uint8))
        text = base64.b64encode(bits.tobytes()).decode()
        lines.append(f"    {K}: (")
        lines += [f'        "{text[i:i + 76]}"' for i in range(0, len(text), 76)]
        lines.append("    ),")
    lines.append("}")
    out = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_had_tables.py")
    with open(out, "w") as f:
        f.write("\n".join(lines) + "\n")
    print(f"wrote {out}")


if __name__ == "__main__":
    main(sys.argv[1])
