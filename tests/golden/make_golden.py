"""Generate the CPU-side golden fixtures from the REFERENCE's own Python oracle.

Run where the reference checkout is available (its location: ``F3S_REFERENCE_DIR``, or the
default below):

    python tests/golden/make_golden.py

It imports ``scripts/tests/test_f3s_accuracy.py`` of the reference with a stub in place of
the compiled ``F3S`` module (the file imports it at the top but the two functions used here
are pure torch), and calls the reference's ``row_wise_softmax_mask`` and ``process_matrix``
on seeded CPU inputs.  The committed ``attention_dense_*.npz`` files hold the inputs and the
reference's outputs; ``tests/test_oracle_attention.py`` checks ``oracle/attention_oracle.py``
against them.  The reference draws Q/K/V with the CUDA generator
(test_f3s_accuracy.py:129-131), which cannot be reproduced on a CPU, so the inputs here are
drawn with the CPU generator from the same seeds and distributions.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types
from pathlib import Path

import numpy as np
import scipy.sparse  # noqa: F401  (the reference script uses ``scipy as sp`` then ``sp.sparse``)
import torch

HERE = Path(__file__).resolve().parent
# the reference checkout: F3S_REFERENCE_DIR, else a directory named "reference" beside this repository
REF = Path(os.environ.get("F3S_REFERENCE_DIR", HERE.parent.parent.parent / "reference"))


def load_reference_script():
    sys.modules.setdefault("F3S", types.ModuleType("F3S"))  # never called
    path = REF / "scripts" / "tests" / "test_f3s_accuracy.py"
    spec = importlib.util.spec_from_file_location("ref_test_f3s_accuracy", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def make_case(ref, name: str, size: int, emb: int, density: float, seed: int, row_stride: int, dist: str):
    np.random.seed(seed)
    torch.manual_seed(seed)
    import scipy as sp

    a = sp.sparse.random(size, size, density=density, format="csr", data_rvs=np.random.rand)
    a.data = np.ceil(a.data, dtype=np.float32)  # test_f3s_accuracy.py:124
    a.sort_indices()
    a_dense = torch.tensor(a.todense())
    draw = torch.rand if dist == "uniform" else torch.randn
    q = draw(size, emb, dtype=torch.float32).to(torch.float16)
    k = draw(size, emb, dtype=torch.float32).to(torch.float16)
    v = draw(size, emb, dtype=torch.float32).to(torch.float16)
    qf, kf, vf = q.float(), k.float(), v.float()
    sddmm = (qf @ kf.T) * a_dense  # :149
    soft = ref.row_wise_softmax_mask(sddmm, a_dense)  # :159
    true = soft @ vf  # :163
    nosoft = sddmm @ vf  # the skip_softmax branch, :161
    tiles8 = ref.process_matrix(sddmm, 16, 8, False)  # :154 for 8-wide TCBs
    tiles16 = ref.process_matrix(sddmm, 16, 8, True)  # :154 for the 16-wide (1tb1rw) family
    np.savez_compressed(
        HERE / f"attention_dense_{name}.npz",
        rowptr=a.indptr.astype(np.int32),
        colidx=a.indices.astype(np.int32),
        q=q.numpy(), k=k.numpy(), v=v.numpy(),
        row_stride=np.int32(row_stride),
        out_softmax=true[::row_stride].numpy(),
        out_nosoftmax=nosoft[::row_stride].numpy(),
        sddmm_tiles8_head=tiles8[: 64 * 128].numpy(),
        sddmm_tiles16_head=tiles16[: 64 * 128].numpy(),
        sddmm_tiles8_sum=np.float64(tiles8.double().sum().item()),
        sddmm_tiles16_sum=np.float64(tiles16.double().sum().item()),
        sddmm_tiles8_len=np.int64(tiles8.numel()),
        sddmm_tiles16_len=np.int64(tiles16.numel()),
    )
    print(name, "nnz", a.nnz, "out", tuple(true.shape))


if __name__ == "__main__":
    ref = load_reference_script()
    # the reference script's own shape (size 1000, d 128, density 0.1, U[0,1)), rows subsampled
    make_case(ref, "n1000_d128_uniform", 1000, 128, 0.1, 0, 8, "uniform")
    # small cases with empty rows, N % 16 != 0, signed inputs
    make_case(ref, "n100_d32_normal", 100, 32, 0.03, 1, 1, "normal")
    make_case(ref, "n257_d64_normal", 257, 64, 0.05, 2, 1, "normal")
