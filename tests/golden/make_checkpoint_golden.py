"""Generate tests/golden/checkpoint_names.json from the reference's own converters.

    python tests/golden/make_checkpoint_golden.py

Needs a checkout of the reference (see oracle/ref_loader.py).  Runs the reference's
processing_OPT / preprocess_175b / processing_HF_GPT on the synthetic checkpoints of
checkpoint_cases.py and stores, per case, every resulting key with its shape and a
position-weighted checksum."""
import importlib
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from oracle import ref_loader  # noqa: E402
import checkpoint_cases as cc  # noqa: E402


def main():
    assert ref_loader.load_reference_model_package() is not None, "reference checkout not found"
    mods = {"processing_OPT": "energonai.utils.checkpointing_opt", "preprocess_175b": "energonai.utils.checkpointing_opt",
            "processing_HF_GPT": "energonai.utils.checkpointing_hf_gpt2"}
    out = {}
    for name, (build, conv) in cc.CASES.items():
        fn = getattr(importlib.import_module(mods[conv]), conv)
        out[name] = cc.summarise(fn(build()))
        print(name, len(out[name]), "entries")
    with open(os.path.join(HERE, "checkpoint_names.json"), "w") as f:
        json.dump(out, f, indent=0)


if __name__ == "__main__":
    main()
