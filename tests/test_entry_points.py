"""The entry points' contracts that need no GPU: the `generate` signature that the reference's validator checks
(scripts/validate_engine.py:160-181), the command line's options, trace_run's argument parsing."""
import inspect

import pytest


def test_generate_has_the_reference_signature():
    from qwenforge_b200.engine import StudentEngine
    sig = inspect.signature(StudentEngine.generate)
    assert list(sig.parameters) == ["self", "prompts", "max_new_tokens", "batch_size", "suite_name"]
    assert sig.parameters["batch_size"].default == 1 and sig.parameters["suite_name"].default is None
    init = inspect.signature(StudentEngine.__init__)
    names = list(init.parameters)
    assert names[1:7] == ["model_path", "device", "dtype", "attn_implementation", "local_files_only", "seed"]
    assert init.parameters["device"].default == "cuda" and init.parameters["attn_implementation"].default == "sdpa"
    assert init.parameters["seed"].default == 0 and init.parameters["local_files_only"].default is False


def test_cli_options_follow_the_reference():
    from qwenforge_b200.cli import parse_args
    args = parse_args(["--model", "some/dir"])
    assert args.device == "cuda" and args.dtype == "bfloat16" and args.attn_implementation == "sdpa"
    assert args.seed == 0 and args.decode_batch_sizes == "1,2,4" and args.ttft_batch_sizes == "1"
    assert args.max_new_tokens_decode == 128 and args.max_new_tokens_ttft == 1
    assert args.warmup_iters == 1 and args.batch_warmup_iters == 0 and args.timed_repeats == 1
    assert not args.local_files_only and not args.verbose_batches
    args = parse_args(["--random-weights", "tiny-a", "--dtype", "float32", "--timed-repeats", "3", "--temperature", "0.7"])
    assert args.random_weights == "tiny-a" and args.timed_repeats == 3 and args.temperature == 0.7
    with pytest.raises(SystemExit):
        parse_args([])                       # neither --model nor --random-weights
    assert parse_args(["--model", "d", "--dtype", "float16"]).dtype == "float16"   # the reference's default name is taken
    args = parse_args(["--model", "d", "--context", "4096", "--prompt-len-range", "64,2048", "--time-kernels"])
    assert args.context == 4096 and args.prompt_len_range == "64,2048" and args.time_kernels


def test_trace_run_arguments():
    from qwenforge_b200.engine.replay import parse_args
    args = parse_args(["--model", "m", "--dtype", "float32", "--out", "o", "--max-tokens", "4096"])
    assert (args.model, args.dtype, args.out, args.max_tokens) == ("m", "float32", "o", 4096)
    with pytest.raises(SystemExit):
        parse_args(["--model", "m", "--dtype", "float16", "--out", "o", "--max-tokens", "64"])
