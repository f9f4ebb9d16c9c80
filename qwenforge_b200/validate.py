"""A standalone check of the entry point's interface, in the manner of the reference's
scripts/validate_engine.py:160-224 (signature of `StudentEngine.generate`, then a two-prompt runtime check).

    python -m qwenforge_b200.validate --model DIR [--device cuda] [--dtype bfloat16] [--attn-implementation sdpa]
    python -m qwenforge_b200.validate --random-weights tiny-b
    python -m qwenforge_b200.validate --skip-load          # the signature alone, no GPU needed

It checks that `generate` has the parameters prompts, max_new_tokens, batch_size and suite_name, that the
constructor takes the reference's keywords, and that two prompts come back as two non-empty strings. The
reference's source scan (forbidden imports and calls) concerns submissions to its course and is not part of this.
"""
from __future__ import annotations

import argparse
import inspect
import sys
import tempfile

GENERATE_PARAMETERS = ("prompts", "max_new_tokens", "batch_size", "suite_name")
CONSTRUCTOR_PARAMETERS = ("model_path", "device", "dtype", "attn_implementation", "local_files_only", "seed")


class ValidationError(Exception):
    pass


def check_signature(cls) -> None:
    if not callable(getattr(cls, "generate", None)):
        raise ValidationError("StudentEngine must define generate().")
    have = inspect.signature(cls.generate).parameters
    for name in GENERATE_PARAMETERS:
        if name not in have:
            raise ValidationError(f"StudentEngine.generate() missing parameter: {name}")
    have = inspect.signature(cls).parameters
    for name in CONSTRUCTOR_PARAMETERS:
        if name not in have:
            raise ValidationError(f"StudentEngine() missing parameter: {name}")


def check_runtime(engine) -> list:
    prompts = ["Say the word one.", "Say the word two."]
    outputs = engine.generate(prompts, max_new_tokens=16, batch_size=2, suite_name="validate")
    if not isinstance(outputs, list):
        raise ValidationError("generate() must return list[str].")
    if len(outputs) != len(prompts):
        raise ValidationError(f"generate() returned {len(outputs)} outputs for {len(prompts)} prompts.")
    if not all(isinstance(item, str) for item in outputs):
        raise ValidationError("Every generate() output must be str.")
    if not all(item.strip() for item in outputs):
        raise ValidationError("Every generate() output must be non-empty for the runtime sanity check.")
    if engine.generate([], max_new_tokens=4) != [] or engine.generate(["x"], max_new_tokens=0) != [""]:
        raise ValidationError("generate() must return [] for no prompts and \"\" for a budget of 0.")
    return outputs


def main(argv=None) -> int:
    p = argparse.ArgumentParser(prog="qwenforge_b200.validate", description=__doc__.split("\n\n")[0])
    p.add_argument("--model", default=None)
    p.add_argument("--random-weights", metavar="PRESET", default=None)
    p.add_argument("--device", default="cuda")
    p.add_argument("--dtype", default="bfloat16")
    p.add_argument("--attn-implementation", default="sdpa")
    p.add_argument("--local-files-only", action="store_true")
    p.add_argument("--skip-load", action="store_true", help="check the signatures only")
    args = p.parse_args(argv)
    from .engine import StudentEngine
    try:
        check_signature(StudentEngine)
        print("Signature check passed.")
        if args.skip_load:
            return 0
        if not args.model and not args.random_weights:
            p.error("give --model DIR or --random-weights PRESET (or --skip-load)")
        holder = None
        model_path = args.model
        if args.random_weights:
            import torch

            from .config import preset_config
            from .weights import write_random_model
            holder = tempfile.TemporaryDirectory(prefix="qf_validate_")
            model_path = holder.name
            write_random_model(preset_config(args.random_weights), 0, model_path,
                               torch.float32 if args.dtype in ("float32", "fp32") else torch.bfloat16)
        try:
            engine = StudentEngine(model_path=model_path, device=args.device, dtype=args.dtype,
                                   attn_implementation=args.attn_implementation, local_files_only=args.local_files_only)
            check_runtime(engine)
        finally:
            if holder is not None:
                holder.cleanup()
        print("Runtime interface check passed.")
        return 0
    except ValidationError as exc:
        print(str(exc), file=sys.stderr)
        return 1


if __name__ == "__main__":
    sys.exit(main())
