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
