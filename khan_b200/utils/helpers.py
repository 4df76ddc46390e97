"""Host-side helpers of the khan front end."""
from __future__ import annotations

import numpy as np


def ed_harder_rmse(y_groups_true, ys_pred) -> float:
    """Relative (conformer-group) RMSE, ``khan/utils/helpers.py:22-68`` of the reference.

    ``y_groups_true`` is a list of groups of true energies, ``ys_pred`` the predictions of all
    groups concatenated.  Inside each group the predictions are shifted so that the prediction at
    the group's lowest TRUE energy equals that energy; the result is the mean over groups of the
    per-group RMSE."""
    sizes = [len(g) for g in y_groups_true]
    pred = np.asarray(ys_pred, dtype=np.float64)
    assert sum(sizes) == len(pred), (sum(sizes), len(pred))
    rmses, start = [], 0
    for g, n in zip(y_groups_true, sizes):
        true = np.asarray(g, dtype=np.float64)
        p = pred[start:start + n]
        lowest = int(np.argmin(true))
        shifted = p + (true[lowest] - p[lowest])
        rmses.append(np.sqrt(np.mean((shifted - true) ** 2)))
        start += n
    return float(np.mean(rmses))
