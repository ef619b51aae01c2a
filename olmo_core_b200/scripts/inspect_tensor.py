"""
Print entries of a distributed checkpoint without loading it whole (role of src/scripts/inspect_tensor.py)::

    python -m olmo_core_b200.scripts.inspect_tensor CHECKPOINT_DIR                 # list keys, shapes, dtypes
    python -m olmo_core_b200.scripts.inspect_tensor CHECKPOINT_DIR model.embeddings.weight [more keys]
"""

import argparse

from ..distributed.checkpoint import get_checkpoint_metadata, load_keys
from ..utils import prepare_cli_environment


def main(argv=None) -> None:
    p = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    p.add_argument("checkpoint_dir")
    p.add_argument("keys", nargs="*")
    args = p.parse_args(argv)
    prepare_cli_environment()
    source = args.checkpoint_dir.rstrip("/")
    if not source.endswith("model_and_optim"):
        source += "/model_and_optim"
    if not args.keys:
        for key, meta in sorted(get_checkpoint_metadata(source).state_dict_metadata.items()):
            size = getattr(meta, "size", None)
            props = getattr(meta, "properties", None)
            print(f"{key}: {tuple(size) if size is not None else type(meta).__name__}"
                  f"{' ' + str(props.dtype) if props is not None else ''}")
        return
    for key, t in zip(args.keys, load_keys(source, args.keys)):
        if hasattr(t, "shape"):
            f = t.float()
            print(f"{key}: shape={tuple(t.shape)} dtype={t.dtype} mean={f.mean():.6g} std={f.std():.6g} "
                  f"min={f.min():.6g} max={f.max():.6g} norm={f.norm():.6g}")
            print(t)
        else:
            print(f"{key}: {t!r}")


if __name__ == "__main__":
    main()
