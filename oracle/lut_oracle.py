"""CPU restatement of the reference's lookup-table (embedding) arithmetic.  TEST INFRASTRUCTURE:
imported by tests/, the smoke check and bench.py's CPU legs only -- never by the product path.

Follows ngraph/transformers/cpu/cpuengine.py:421-435 (fprop_lut, update_lut), the code the
reference's CPU transformer runs; pinned against that transformer through the fixture
tests/golden/fixtures/lut_embedding.npz.
"""
import numpy as np


def lut_fprop(lut, idx, axis):
    """lut: 2-d table, idx: 1-d indices (any numeric dtype) -> lut.take(idx, axis)
    (cpuengine.py:421-422)."""
    return lut.take(np.asarray(idx).astype(int), axis)


def lut_update(error, idx, pad_idx, axis, table_shape):
    """Gradient of the table: for every index that occurs, the sum of the rows (axis 0) or columns
    (axis 1) of `error` at the positions where it occurs; pad_idx and unused rows stay zero
    (cpuengine.py:425-435)."""
    dW = np.zeros(table_shape, dtype=np.float32)
    idx = np.asarray(idx).astype(int)
    for w in np.unique(idx):
        if pad_idx is not None and w == pad_idx:
            continue
        where = np.where(idx == w)[0]
        total = np.sum(error.take(where, axis=axis), axis=axis)
        if axis == 0:
            dW[w, :] = total
        else:
            dW[:, w] = total
    return dW
