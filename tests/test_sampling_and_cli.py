"""Sampling options, random streams and the command line's argument handling (no GPU).
The option cases follow the reference's own sampler tests (tests/unit/sampler.test.ts)."""
import pytest

from binfer_b200.cli import CliError, parse_args, pre_parse
from binfer_b200.sampling import SamplingParams, uniform


def test_defaults_are_the_command_lines():
    p = SamplingParams()
    assert (p.temperature, p.top_k, p.top_p, p.repetition_penalty, p.max_tokens) == \
        (0.0, 0, 1.0, 1.0, 100)
    assert p.greedy and isinstance(p.seed, int)


@pytest.mark.parametrize("bad", [dict(temperature=-1), dict(top_k=-2), dict(top_p=0.0),
                                 dict(top_p=1.5), dict(repetition_penalty=0), dict(max_tokens=0)])
def test_bad_options_are_refused(bad):
    with pytest.raises(ValueError):
        SamplingParams(**bad)


def test_uniform_stream_is_a_function_of_seed_and_index():
    a = [uniform(7, n) for n in range(2000)]
    assert a == [uniform(7, n) for n in range(2000)]
    assert a != [uniform(8, n) for n in range(2000)]
    assert all(0.0 <= u < 1.0 for u in a)
    assert 0.45 < sum(a) / len(a) < 0.55
    assert len(set(a)) > 1990


def test_unknown_flag_is_refused_before_anything_loads(capsys):
    assert pre_parse(["model", "--no-such-flag"]) == 1
    assert "Unknown flag '--no-such-flag'" in capsys.readouterr().err
    assert pre_parse(["-h"]) == 0
    assert "--max-tokens" in capsys.readouterr().out
    assert pre_parse(["model", "--temperature", "-0.5", "--top-k", "5"]) is None


def test_arguments_with_the_references_names_and_defaults():
    a = parse_args(["/m", "1,2,3"])
    assert a["model"] == "/m" and a["prompt"] == "1,2,3"
    assert (a["max_tokens"], a["temperature"], a["top_k"], a["top_p"]) == (100, 0.0, 0, 1.0)
    assert a["cuda_graphs"] and a["tp"] == "auto" and not a["bench"]
    b = parse_args(["/m", "-p", "4 5", "--max-tokens", "7", "--temp", "0.8", "--top-k", "40",
                    "--top-p", "0.9", "--no-cuda-graphs", "--dtype", "fp32", "-q", "--bench",
                    "--profile", "--tp", "1", "--no-cache"])
    assert (b["prompt"], b["max_tokens"], b["temperature"], b["top_k"], b["top_p"]) == \
        ("4 5", 7, 0.8, 40, 0.9)
    assert not b["cuda_graphs"] and b["dtype"] == "fp32" and b["quiet"] and b["bench"] and b["profile"]


@pytest.mark.parametrize("argv", [[], ["/m", "--tp", "2"], ["/m", "--dtype", "fp16"],
                                  ["/m", "-i", "in.txt"], ["/m", "--max-tokens", "x"]])
def test_bad_command_lines(argv):
    with pytest.raises(CliError):
        parse_args(argv)
