"""Operator KEY=VALUE configuration -> command line (CPU only)."""
import pytest

from cuteafd_b200 import cli, configfile
from cuteafd_b200.configfile import ConfigError


def test_example_config_becomes_a_serve_command(capsys):
    assert cli.main(["run", "--config", "examples/configs/qwen3-235b-1gpu.config", "--set", "listen=0.0.0.0:9000", "--set", "DRAFT=off", "--print"]) == 0
    line = capsys.readouterr().out.strip()
    assert line.startswith("cuteafd serve --model qwen3-235b --listen 0.0.0.0:9000") and "--host-cache-gib 64" in line
    assert "--draft off" in line and "--usage on" in line and "--official-model-names gpt-4o,claude-sonnet-4" in line


def test_parsing_rules():
    cfg = configfile.parse_text('A=1\n# c\n\nB="x y"   \nC=${A}-${ENV:HOME_X} # tail\nD=v # comment\n')
    assert cfg == {"A": "1", "B": "x y", "C": "${A}-${ENV:HOME_X}", "D": "v"}
    assert configfile.expand(cfg, env={"HOME_X": "h"})["C"] == "1-h"
    with pytest.raises(ConfigError, match="not set"):
        configfile.expand(cfg, env={})
    with pytest.raises(ConfigError, match="KEY=VALUE"):
        configfile.parse_text("just words")
    with pytest.raises(ConfigError, match="retired; use MODEL"):
        configfile.parse_text("SNAPSHOT=/x")
    with pytest.raises(ConfigError, match="retired; use DRAFT"):
        configfile.apply_overrides({}, ["speculator=mtp"])
    with pytest.raises(ConfigError, match="loop"):
        configfile.expand({"A": "${B}", "B": "${A}"})


def test_unknown_keys_booleans_and_choices(tmp_path, capsys):
    f = tmp_path / "c.config"
    f.write_text("COMMAND=serve\nENABLE_BENCH=true\nMAX_SEQUENCE=4\n")
    assert cli.main(["run", "--config", str(f), "--print"]) == 2
    assert "did you mean MAX_SEQUENCES" in capsys.readouterr().err
    f.write_text("COMMAND=serve\nENABLE_BENCH=yes\nDRAFT=ngram\n")
    assert cli.main(["run", "--config", str(f), "--print"]) == 0
    assert capsys.readouterr().out.strip() == "cuteafd serve --enable-bench --draft ngram"
    f.write_text("ENABLE_BENCH=off\nDRAFT=psychic\n")
    assert cli.main(["run", "--config", str(f), "--print"]) == 2 and "expected one of" in capsys.readouterr().err
    f.write_text("COMMAND=teleport\n")
    assert cli.main(["run", "--config", str(f), "--print"]) == 2
