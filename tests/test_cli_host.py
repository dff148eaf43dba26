"""The command line's host side: option names of the reference, precedence, .env parsing."""
import json
import os

import pytest

from llm_infer_engine_b200.cli import main as cli


def test_option_names_follow_the_reference():
    p = cli.build_parser()
    flags = {a for action in p._actions for a in action.option_strings}
    for flag in ("--env-file", "--tokenizer", "--weights", "--prompt", "--prompt-file", "--system-prompt",
                 "--max-new-tokens", "--temperature", "--top-p", "--device", "--seed", "--dim", "--n-layers",
                 "--n-heads", "--n-kv-heads", "--hidden-dim", "--vocab-size", "--max-seq-len", "--cuda-graph"):
        assert flag in flags, flag
    assert "--quantization" not in flags


def test_env_file_and_precedence(tmp_path, monkeypatch):
    env = tmp_path / ".env"
    env.write_text("# comment\nexport LLM_TEMPERATURE=0.5\nLLM_TOP_P='0.8'\nLLM_PROMPT=\"hi there\"\nnoequals\nLLM_SEED=\n")
    data = cli.parse_env_file(str(env))
    assert data == {"LLM_TEMPERATURE": "0.5", "LLM_TOP_P": "0.8", "LLM_PROMPT": "hi there", "LLM_SEED": ""}
    assert cli.parse_env_file(str(tmp_path / "missing")) == {}
    monkeypatch.setenv("LLM_TEMPERATURE", "0.9")
    monkeypatch.setenv("LLM_MAX_NEW_TOKENS", "17")
    args = cli.build_parser().parse_args(["--top-p", "0.6"])
    opts = cli.resolve_all(args, data)
    assert opts["top_p"] == 0.6                     # command line first
    assert opts["temperature"] == 0.5               # then the .env file
    assert opts["max_new_tokens"] == 17             # then the environment
    assert opts["seed"] is None                     # an empty value is no value
    assert opts["system_prompt"] == "You are a helpful assistant." and opts["max_seq_len"] == 4096
    assert opts["prompt"] == "hi there"


def test_device_and_random_config():
    assert cli.device_index("cuda") == 0 and cli.device_index("cuda:3") == 3 and cli.device_index("2") == 2
    with pytest.raises(ValueError, match="CUDA"):
        cli.device_index("cpu")
    args = cli.build_parser().parse_args(["--dim", "64", "--n-layers", "2", "--n-heads", "4", "--hidden-dim", "128"])
    opts = cli.resolve_all(args, {})
    with pytest.raises(ValueError, match="--vocab-size"):
        cli.config_from_flags(opts)
    opts["vocab_size"] = 100
    cfg = cli.config_from_flags(opts)
    assert cfg["hidden_size"] == 64 and cfg["num_key_value_heads"] == 4 and cfg["vocab_size"] == 100


def test_prepare_model_folder(tmp_path):
    import plain_llama as plain
    from llm_infer_engine_b200 import write_random_model
    real = write_random_model(plain.TINY_A, str(tmp_path / "real"), seed=0)
    base = cli.resolve_all(cli.build_parser().parse_args([]), {})
    assert cli.prepare_model_folder(dict(base, model=real), log=lambda s: None) == real
    # --weights FILE with config.json beside the tokenizer, as the reference is called
    tok = tmp_path / "tok"
    tok.mkdir()
    (tok / "config.json").write_text(json.dumps(plain.TINY_A))
    folder = cli.prepare_model_folder(dict(base, tokenizer=str(tok), weights=os.path.join(real, "model.safetensors")),
                                      log=lambda s: None)
    assert os.path.samefile(os.path.join(folder, "model.safetensors"), os.path.join(real, "model.safetensors"))
    # no weights: random weights from the config.json found
    folder = cli.prepare_model_folder(dict(base, tokenizer=str(tok), seed=3), log=lambda s: None)
    assert os.path.isfile(os.path.join(folder, "model.safetensors"))
    with pytest.raises(FileNotFoundError):
        cli.prepare_model_folder(dict(base, tokenizer=str(tok), weights="/no/such/file"), log=lambda s: None)


def test_prompt_ids_file_and_init_std(tmp_path):
    ids = tmp_path / "ids.txt"
    ids.write_text("5, 17 3\n9,\n")
    assert cli.read_ids_file(str(ids)) == "5,17,3,9"
    ids.write_text("5 x")
    with pytest.raises(ValueError, match="not a token id"):
        cli.read_ids_file(str(ids))
    args = cli.build_parser().parse_args(["--init-std", "0.05", "--prompt-ids-file", str(ids)])
    opts = cli.resolve_all(args, {})
    assert opts["init_std"] == 0.05 and opts["prompt_ids_file"] == str(ids)
    assert cli.resolve_all(cli.build_parser().parse_args([]), {})["init_std"] == 0.02
