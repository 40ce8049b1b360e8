"""The command line's names, defaults and refusals, without a GPU: everything up to the point where the
engine would be built.  Names and defaults are the reference launcher's where it has them
(llama-tornado:330-492 and Options.java:31-48, 103-114 of the reference project)."""
import json

import pytest

from gpullama3.java_b200.engine import cli


def parse(*argv):
    return cli.create_parser().parse_args(list(argv))


def test_defaults_are_the_reference_launchers():
    a = parse("--model", "m", "--prompt", "1 2 3")
    assert a.temperature == pytest.approx(0.1) and a.top_p == pytest.approx(0.95)    # Options.java:14-15
    assert a.max_tokens == 512 and a.seed is None                                    # seed: the clock, chosen at run time
    assert a.stream is True and a.echo is False
    assert a.instruct is True and a.interactive is False and a.use_gpu is True
    assert a.dtype == "bfloat16"


def test_short_and_long_names_mean_the_same():
    long = parse("--model", "m", "--prompt", "1,2", "--max-tokens", "7", "--temperature", "0", "--seed", "5", "--system-prompt", "9")
    short = parse("-m", "m", "-p", "1 2", "-n", "7", "--temp", "0", "-s", "5", "-sp", "9")
    assert vars(long) == vars(short)
    assert long.prompt == [[1, 2]] and long.system_prompt == [9]
    assert parse("-m", "m", "-p", "1", "--chat").interactive and parse("-m", "m", "-p", "1", "-i").interactive


def test_prompts_are_token_ids_and_repeat_into_a_batch():
    a = parse("-m", "m", "-p", "5 6 7", "-p", "8,9")
    assert a.prompt == [[5, 6, 7], [8, 9]]
    with pytest.raises(SystemExit):
        parse("-m", "m", "-p", "hello world")      # no tokenizer here: text is refused with a message
    with pytest.raises(SystemExit):
        parse("-m", "m", "-p", " ")
    with pytest.raises(SystemExit):
        parse("-m", "m", "-p", "1", "--stream", "maybe")
    assert parse("-m", "m", "-p", "1", "--stream", "false").stream is False


@pytest.mark.parametrize("argv", [
    ["-m", "m", "-p", "1", "--interactive"],                       # chat needs a tokenizer
    ["-m", "m", "-p", "1", "--suffix", "x"],                       # fill-in-the-middle is not built
    ["-m", "m", "-p", "1", "--temperature", "-0.5"],               # Options.java:71
    ["-m", "m", "-p", "1", "--top-p", "1.5"],                      # Options.java:72
    ["-p", "1"],                                                   # neither a model nor random weights
    ["-m", "m", "--config", "c.json", "--random-weights", "1", "-p", "1"],   # both
    ["--random-weights", "1", "-p", "1"],                          # random weights of which configuration?
    ["-m", "m"],                                                   # no prompt
])
def test_refusals_come_before_any_model_is_built(argv, capsys):
    with pytest.raises(SystemExit) as e:
        cli.main(argv + ["--show-command"])
    assert e.value.code == 2
    assert "error" in capsys.readouterr().err


def test_show_command_prints_what_would_run_and_stops(tmp_path, capsys):
    prompts = tmp_path / "prompts.txt"
    prompts.write_text("1 2 3\n\n4,5\n")
    rc = cli.main(["-m", "some/folder", "-p", "7 8", "--prompt-file", str(prompts), "-sp", "100", "-n", "10", "--seed", "3",
                   "--max-batch", "2", "--show-command"])
    assert rc == 0
    shown = json.loads(capsys.readouterr().out)
    assert shown["model"] == "some/folder" and shown["prompts"] == 3 and shown["seed"] == 3
    assert shown["temperature"] == pytest.approx(0.1) and shown["top_p"] == pytest.approx(0.95)
    # the cache holds the first batch: two prompts of 3 and 4 tokens (system token included) plus 10 new tokens each,
    # each request rounded up to a page of 64
    assert shown["cache_tokens"] == 128 and shown["max_batch"] == 2
    rc = cli.main(["-m", "x", "-p", "1", "--cache-tokens", "4096", "--show-command"])
    assert rc == 0 and json.loads(capsys.readouterr().out)["cache_tokens"] == 4096


def test_position_cap_profile_and_bench_switches_exist():
    a = parse("-m", "m", "-p", "1", "--max-len", "300", "--profile", "--bench", "--norm-std", "0.1")
    assert a.max_len == 300 and a.profile and a.bench and a.norm_std == pytest.approx(0.1)
    b = parse("-m", "m", "-p", "1")
    assert b.max_len is None and not b.profile and not b.bench and not b.show_config


def test_show_config_prints_the_typed_configuration(tmp_path, capsys):
    from conftest import TINY_B

    (tmp_path / "config.json").write_text(json.dumps(TINY_B))
    assert cli.main(["-m", str(tmp_path), "-p", "1", "--show-config"]) == 0
    shown = json.loads(capsys.readouterr().out)
    assert shown["config"]["num_key_value_heads"] == 1 and shown["config"]["rope_scaling"]["factor"] == 8.0
    assert shown["q_dim"] == 96 and shown["kv_dim"] == 32 and shown["layers"] == 3
    assert shown["parameters"] == 369312                     # the count BASELINE's Tiny B implies
    assert shown["max_sequence_length"] == 256 and shown["stop_token_ids"] == [3, 5]
    assert cli.main(["--config", str(tmp_path / "config.json"), "--random-weights", "1", "-p", "1", "--show-config"]) == 0


def test_stop_ids_come_from_generation_config_when_it_has_them(tmp_path):
    from conftest import TINY_A
    from gpullama3.java_b200.config import config_from_dict
    from gpullama3.java_b200.engine.api import read_stop_ids

    cfg = config_from_dict(TINY_A)
    assert read_stop_ids(tmp_path, cfg) == (7,)                                  # config.json's eos_token_id
    (tmp_path / "generation_config.json").write_text(json.dumps({"temperature": 0.6}))
    assert read_stop_ids(tmp_path, cfg) == (7,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": [11, 12, 13]}))
    assert read_stop_ids(tmp_path, cfg) == (11, 12, 13)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": 9}))
    assert read_stop_ids(tmp_path, cfg) == (9,)
    (tmp_path / "generation_config.json").write_text(json.dumps({"eos_token_id": "x"}))
    with pytest.raises(ValueError):
        read_stop_ids(tmp_path, cfg)


def test_profile_table_lists_the_longest_first():
    table = cli.format_profile({"b200_rmsnorm": (4, 0.02), "b200_gemm_generic": (10, 1.5)})
    lines = table.splitlines()
    assert lines[1].startswith("b200_gemm_generic") and lines[2].startswith("b200_rmsnorm") and "98.7%" in lines[1]
