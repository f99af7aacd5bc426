"""Front-to-back tuning of the per-layer thresholds, the procedure the reference describes in its readme
(readme.md:193-214): walk the registry ``DCThreshold.t`` in registration (= forward) order and raise each layer's
threshold geometrically until the loss over a calibration sequence exceeds what it was before that layer was
touched by more than the allowed factor; keep the last value that stayed inside. The result is saved in the JSON
format ``DCThreshold.load_thresholds`` reads (src/deltacnn/sparse_layers.py:159-186)."""
from .sparse_layers import DCThreshold


def tune_thresholds(calc_loss, keys=None, start=1e-3, step=2.0, max_loss_increase=1.001, abs_slack=0.0, max_threshold=4.0,
                    log=None):
    """``calc_loss()`` runs the calibration sequence through the model (from a reset state) with the thresholds
    currently in ``DCThreshold.t`` and returns a non-negative loss. ``keys`` defaults to every registered layer, in
    order. A layer may raise the loss from ``L`` (measured before it is touched) to at most
    ``max(L * max_loss_increase, L + abs_slack)``; ``abs_slack`` matters when the loss starts at exactly zero.
    Returns the list of chosen thresholds in registration order."""
    keys = list(DCThreshold.t.keys()) if keys is None else list(keys)
    for i, key in enumerate(keys):
        before = calc_loss()
        budget = max(before * max_loss_increase, before + abs_slack)
        value, accepted = start, 0.0
        while value <= max_threshold:
            DCThreshold.t[key] = value
            loss = calc_loss()
            if loss > budget:
                break
            accepted = value
            value *= step
        DCThreshold.t[key] = accepted
        if log is not None:
            log(f"layer {i}: threshold {accepted:g} (loss {before:.6g} -> budget {budget:.6g})")
    return [DCThreshold.t[k] for k in DCThreshold.t.keys()]
