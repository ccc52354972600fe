"""Stage the reference's own Python for the hot path under oracle/_ref/.  TEST INFRASTRUCTURE ONLY.

    python oracle/make_ref.py --reference /path/to/landmark-attention

The reference (epfml/landmark-attention) is pure Python: there is nothing to compile.  This recipe copies, unmodified,
the few files its hot path lives in from a checkout into oracle/_ref/ (git-ignored: the copies never enter this
repository's history), so that the benchmark's reference arm and CPU baseline can time the reference's own code on a
machine where the checkout itself is absent:

  llama/llama_mem.py, llama/llama_landmark_config.py      high-level grouped softmax + LLaMA retrieval branch
  llama/ltriton/flash_landmark_attention.py               the reference's fused kernels (Triton)
  lm_benchmark/models/{landmark.py, caches/, positional_encoders/}   lm_benchmark attention, block cache, rotary

Nothing under landmark_attention_b200/ imports these files.
"""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF_DIR = os.path.join(HERE, "_ref")
FILES = [
    "llama/llama_mem.py",
    "llama/llama_landmark_config.py",
    "llama/ltriton/flash_landmark_attention.py",
    "lm_benchmark/models/landmark.py",
    "lm_benchmark/models/caches/__init__.py",
    "lm_benchmark/models/caches/cache.py",
    "lm_benchmark/models/caches/kv_cache.py",
    "lm_benchmark/models/caches/kv_cache_train.py",
    "lm_benchmark/models/caches/mem_cache.py",
    "lm_benchmark/models/positional_encoders/__init__.py",
    "lm_benchmark/models/positional_encoders/encoder.py",
    "lm_benchmark/models/positional_encoders/rotary.py",
    "lm_benchmark/models/positional_encoders/rotary_mem_jump.py",
    "lm_benchmark/models/positional_encoders/rotary_utils.py",
]


def stage(reference: str) -> str:
    """Copy FILES from the checkout at `reference` into oracle/_ref/ (same relative paths); returns that folder."""
    missing = [f for f in FILES if not os.path.isfile(os.path.join(reference, f))]
    if missing:
        raise FileNotFoundError(f"not a landmark-attention checkout ({reference}): missing {missing}")
    for f in FILES:
        dst = os.path.join(REF_DIR, f)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(os.path.join(reference, f), dst)
    # lm_benchmark/models/__init__.py of the checkout imports model files that are not staged; an empty package
    # marker is enough for `models.landmark` to import its siblings
    open(os.path.join(REF_DIR, "lm_benchmark", "models", "__init__.py"), "w").close()
    return REF_DIR


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of an epfml/landmark-attention checkout")
    a = ap.parse_args()
    print(stage(a.reference))
    sys.exit(0)
