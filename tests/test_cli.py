"""The command line's parsing, on the CPU (src/cli/args.cpp's rules; tests/cli/test_args.cpp in spirit)."""
import json

import pytest

import plain_qwen3 as plain
from tiny_inference_engine_b200.cli.main import main, parse_ids, parse_size
from tiny_inference_engine_b200.errors import InvalidArgument


def test_sizes():
    assert parse_size("4G") == 4 << 30 and parse_size("512m") == 512 << 20 and parse_size("16K") == 16384
    assert parse_size("1000") == 1000
    for bad in ("", "G", "1.5G", "-1", "0", "12X"):
        with pytest.raises(InvalidArgument):
            parse_size(bad)


def test_ids():
    assert parse_ids("1 2,3 ,4") == [1, 2, 3, 4] and parse_ids("") == []
    with pytest.raises(InvalidArgument):
        parse_ids("1 two")


def test_usage_and_errors(capsys, tmp_path):
    assert main([]) == 1 and "usage: tie generate" in capsys.readouterr().err
    assert main(["--help"]) == 0 and "--kv-mem" in capsys.readouterr().out
    assert main(["serve"]) == 1 and "unknown command 'serve'" in capsys.readouterr().err
    assert main(["generate", "-p", "1 2"]) == 1 and "--model is required" in capsys.readouterr().err
    assert main(["generate", "-m", "x"]) == 1 and "exactly one of" in capsys.readouterr().err
    assert main(["generate", "-m", "x", "-p", "1", "--device", "metal"]) == 1 and "must be cuda" in capsys.readouterr().err
    assert main(["generate", "-m", "x", "-p", "1", "--temp", "-1"]) == 1 and "temperature" in capsys.readouterr().err
    assert main(["generate", "-m", "x", "-p", "1", "--top-p", "0"]) == 1 and "top_p" in capsys.readouterr().err


def test_make_random_writes_a_folder(tmp_path, capsys):
    cfg = tmp_path / "c.json"
    cfg.write_text(json.dumps(plain.TINY_A))
    assert main(["make-random", "-o", str(tmp_path / "m"), "--config", str(cfg), "--seed", "3", "--dtype", "float32"]) == 0
    assert (tmp_path / "m" / "model.safetensors").exists() and (tmp_path / "m" / "config.json").exists()
