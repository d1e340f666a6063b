"""Generates ``tests/golden/event_golden.npz``.

Connectivity fixtures come from the reference's own generator calls
(``brainstate/nn/_event_fixedprob.py:165-171,183-190``: NumPy ``RandomState``),
which is the only part of the path that can be executed in a container without
JAX/brainevent.  Product fixtures are computed the way the reference's tests
recompute their oracles (``brainstate/nn/_event_fixedprob_test.py:77-81,254-259``):
a Python loop over presynaptic rows with ``np.add.at`` in float32, written here
independently of ``oracle/``.  The dense-event known-answer case restates
``brainstate/nn/_event_linear_test.py:126-162``.

Run from the repository root:  python tests/golden/make_golden.py
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def scatter_ref(x, indices, w, n_post, homo):
    ref = np.zeros((n_post,), np.float32)
    for i in range(indices.shape[0]):
        np.add.at(ref, indices[i], np.float32((w if homo else w[i]) * np.float32(x[i])))
    return ref


def main():
    out = {}
    cases = [(123, 20, 40, 4), (11, 20, 30, 6), (7, 33, 1000, 17), (5, 64, 128, 128)]
    for c, (seed, n_pre, n_post, K) in enumerate(cases):
        rng = np.random.RandomState(seed)
        idx = rng.randint(0, n_post, size=(n_pre, K)).astype(np.int32)
        sel = rng.random(n_pre) < 0.5                                   # the afferent_ratio mask
        r2 = np.random.RandomState(1000 + seed)
        spk = r2.random_sample(n_pre) < 0.3
        xf = (r2.random_sample(n_pre) * spk).astype(np.float32)          # float input, zeros where silent
        w_het = r2.uniform(-1, 1, size=(n_pre, K)).astype(np.float32)
        ct = r2.standard_normal(n_post).astype(np.float32)
        out[f'c{c}_meta'] = np.array([seed, n_pre, n_post, K], np.int64)
        out[f'c{c}_indices'] = idx
        out[f'c{c}_pre_selected'] = sel
        out[f'c{c}_spk'] = spk
        out[f'c{c}_xf'] = xf
        out[f'c{c}_w_het'] = w_het
        out[f'c{c}_ct'] = ct
        out[f'c{c}_y_event_homo'] = scatter_ref(spk.astype(np.float32), idx, np.float32(1.5), n_post, True)
        out[f'c{c}_y_event_het'] = scatter_ref(spk.astype(np.float32), idx, w_het, n_post, False)
        out[f'c{c}_y_float_het'] = scatter_ref(xf, idx, w_het, n_post, False)
        # transpose product and weight cotangent for y = x @ W, output cotangent ct
        dx = np.array([np.sum((w_het[i] * ct[idx[i]]).astype(np.float64)) for i in range(n_pre)], np.float32)
        out[f'c{c}_dx_het'] = dx
        out[f'c{c}_dw_het_float'] = (xf[:, None] * ct[idx]).astype(np.float32)
        out[f'c{c}_dw_het_event'] = (spk[:, None].astype(np.float32) * ct[idx]).astype(np.float32)
        out[f'c{c}_dw_homo_event'] = np.float32(np.sum((spk[:, None] * ct[idx]).astype(np.float64)))
    # dense event known answer
    out['dense_spk'] = np.array([0, 2, 0, 3, 0, 0, 1, 0, 0, 5], np.float32)
    out['dense_w'] = np.float32(1.5)
    out['dense_event_true'] = np.float32(4 * 1.5)
    out['dense_event_false'] = np.float32(11 * 1.5)
    np.savez_compressed(os.path.join(HERE, 'event_golden.npz'), **out)
    print('wrote', os.path.join(HERE, 'event_golden.npz'), len(out), 'arrays')


if __name__ == '__main__':
    main()
