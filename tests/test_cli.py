"""The command line's options (no GPU needed): names, defaults and TESSERACT_* fallbacks of the reference's binary
(src/config.rs:139-186), plus what this command adds for generation."""

import importlib


def fresh_cli(monkeypatch, env):
    for key in ("MODEL_PATH", "DEVICE", "MAX_QUEUE", "MAX_RUNNING", "MAX_BATCH_TOKENS", "PREFILL_CHUNK_TOKENS",
                "MAX_SEQUENCE_LENGTH", "KV_CAPACITY_TOKENS"):
        monkeypatch.delenv("TESSERACT_" + key, raising=False)
    for key, value in env.items():
        monkeypatch.setenv("TESSERACT_" + key, value)
    import tesseract_b200.cli as cli

    return importlib.reload(cli)


def test_defaults_are_the_reference_servers(monkeypatch):
    args = fresh_cli(monkeypatch, {}).build_parser().parse_args(["--model-path", "m"])
    assert (args.max_queue, args.max_running, args.max_batch_tokens, args.prefill_chunk_tokens) == (256, 32, 4096, 512)
    assert (args.max_sequence_length, args.kv_capacity_tokens, args.device) == (131072, 32768, 0)
    assert (args.max_tokens, args.temperature, args.top_p, args.seed) == (128, 1.0, 1.0, None)
    assert args.dtype == "bfloat16" and not args.check_weights and not args.no_cuda_graphs


def test_environment_fallbacks_and_flags_over_them(monkeypatch):
    cli = fresh_cli(monkeypatch, {"MODEL_PATH": "/models/x", "MAX_RUNNING": "7", "KV_CAPACITY_TOKENS": "4096"})
    args = cli.build_parser().parse_args([])
    assert args.model_path == "/models/x" and args.max_running == 7 and args.kv_capacity_tokens == 4096
    args = cli.build_parser().parse_args(["--max-running", "3", "--check-weights", "--prompt-ids", "1,2", "--prompt-ids", "3"])
    assert args.max_running == 3 and args.check_weights and args.prompt_ids == ["1,2", "3"]


def test_missing_model_or_config_is_refused_before_anything_is_loaded(monkeypatch, capsys):
    cli = fresh_cli(monkeypatch, {})
    assert cli.main([]) == 2
    assert "--model-path" in capsys.readouterr().err
    assert cli.main(["--random-weights", "3"]) == 2
    assert "--config" in capsys.readouterr().err
