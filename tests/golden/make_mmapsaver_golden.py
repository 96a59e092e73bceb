"""Generates ``mmapsaver_*.mmap``: stores written by the UNMODIFIED reference ``MmapSaver``
(trak/savers.py:241-457) for a tiny checkpoint, filled with known values.

    python tests/golden/make_mmapsaver_golden.py --reference /path/to/trak

They pin the byte layout that ``trak_b200/mmap_io.py`` has to read and reproduce.
"""
import argparse
import logging
import os
import shutil
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
N, K, M = 6, 8, 3


def values(shape, dtype, offset=0.0):
    return (np.arange(np.prod(shape), dtype=np.float64).reshape(shape) / 8.0 - 2.0 + offset).astype(dtype)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of MadryLab/trak")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    from trak.savers import MmapSaver

    for half, tag in ((True, "f16"), (False, "f32")):
        tmp = tempfile.mkdtemp()
        try:
            saver = MmapSaver(save_dir=tmp, metadata={"JL dimension": K, "JL matrix type": "rademacher",
                                                      "train set size": N},
                              train_set_size=N, proj_dim=K, load_from_save_dir=True,
                              logging_level=logging.WARNING, use_half_precision=half)
            saver.register_model_id(0, _allow_featurizing_already_registered=False)
            dt = np.float16 if half else np.float32
            saver.current_store["grads"][:] = values((N, K), dt)
            saver.current_store["features"][:] = values((N, K), dt, 0.5)
            saver.current_store["out_to_loss"][:] = values((N, 1), dt, 1.0)
            for v in saver.current_store.values():
                v.flush()
            saver.init_experiment("exp", M, 0)
            saver.current_store["exp_scores"][:] = values((N, M), dt, 0.25)
            saver.current_store["exp_scores"].flush()
            for src, dst in (("0/grads.mmap", f"mmapsaver_grads_{tag}.mmap"),
                             ("0/features.mmap", f"mmapsaver_features_{tag}.mmap"),
                             ("0/out_to_loss.mmap", f"mmapsaver_out_to_loss_{tag}.mmap"),
                             ("scores/exp.mmap", f"mmapsaver_scores_{tag}.mmap")):
                shutil.copyfile(os.path.join(tmp, src), os.path.join(HERE, dst))
        finally:
            shutil.rmtree(tmp, ignore_errors=True)
    print(sorted(f for f in os.listdir(HERE) if f.startswith("mmapsaver_")))


if __name__ == "__main__":
    main()
