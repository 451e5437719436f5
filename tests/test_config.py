import dataclasses
import os

import pytest

from titan_b200.config import configs
from titan_b200.config.manager import ConfigManager, apply_overrides, resolve_recipe


def test_defaults_cover_reference_extension_fields():
    c = configs.TrainerConfig()
    assert c.optimizer.swap_optimizer is False and c.optimizer.swap_optimizer_times == 16
    assert c.optimizer.muon_momentum == 0.95 and c.optimizer.muon_ns_steps == 5
    assert c.optimizer.muon_adjust_lr_fn == "match_rms_adamw"
    assert c.parallelism.context_parallel_load_balancer is None
    assert c.training.num_mtp_modules == 0 and c.training.mtp_loss_weight == 0.3
    assert c.profiling.profile_ranks == [-1] and c.profiling.enable_online_parse
    assert c.checkpoint.sync_files and not c.checkpoint.drop_page_cache_after_save
    assert c.checkpoint.empty_cache_after_save


def test_base_recipes_compose():
    base = configs.trainer_base_config()
    assert base.optimizer.swap_optimizer and base.activation_checkpoint.mode == "full"
    dbg = configs.debug_single_node_eq_pruned_config(base)
    assert dbg.debug.moe_force_load_balance and dbg.training.steps == 20 and dbg.checkpoint.load_only
    cpt = configs.cpt_default_config(base)
    assert cpt.checkpoint.initial_load_in_hf and cpt.comm.trace_buf_size == 0
    sft = configs.sft_default_config(base)
    assert sft.checkpoint.export_dtype == "bfloat16" and sft.training.steps == 100
    # the base is untouched by derived recipes
    assert base.training.steps == 10000


def test_deep_replace_does_not_share_lists():
    base = configs.TrainerConfig()
    other = configs.deep_replace(base)
    other.profiling.profile_ranks.append(3)
    assert base.profiling.profile_ranks == [-1]


def test_cli_overrides():
    cfg = ConfigManager().parse_args([
        "--module", "llama3", "--config", "llama3_debugmodel", "--training.steps", "2", "--checkpoint.enable",
        "--checkpoint.no-sync-files", "--profiling.profile_ranks", "0,1", "--optimizer.lr=0.5",
        "--parallelism.context-parallel-load-balancer", "none", "--checkpoint.async_mode", "async",
    ])
    assert cfg.training.steps == 2 and cfg.checkpoint.enable and cfg.checkpoint.sync_files is False
    assert cfg.profiling.profile_ranks == [0, 1] and cfg.optimizer.lr == 0.5
    assert cfg.parallelism.context_parallel_load_balancer is None
    assert cfg.checkpoint.async_mode == "async"


def test_cli_rejects_unknown_and_bad_literal():
    cfg = resolve_recipe("llama3", "llama3_debugmodel")
    with pytest.raises(KeyError):
        apply_overrides(cfg, ["--training.nope", "1"])
    with pytest.raises(ValueError):
        apply_overrides(cfg, ["--checkpoint.async_mode", "sometimes"])


def test_unknown_recipe_lists_available():
    with pytest.raises(AttributeError, match="llama3_debugmodel"):
        resolve_recipe("llama3", "does_not_exist")


def test_to_dict_is_plain():
    d = configs.TrainerConfig().to_dict()
    assert d["training"]["seq_len"] == 2048 and isinstance(d["profiling"]["profile_ranks"], list)
    assert dataclasses.is_dataclass(configs.TrainerConfig())


def test_union_sections_switch_with_a_variant_token():
    from titan_b200.config.configs import ChatDataLoaderConfig, DSV4EncoderConfig
    from titan_b200.config.manager import ConfigManager

    cfg = ConfigManager().parse_args([
        "--module", "deepseek_v4", "--config", "debug_deepseek_v4_single_node_1b", "--training.seq_len", "1152",
        "dataloader:chat_data_loader_config", "--dataloader.dataset_path", "parquet", "--dataloader.data_files", "a.parquet",
        "dataloader.chat_encoder:dsv4_encoder_config", "--dataloader.chat_encoder.mode", "thinking"])
    assert isinstance(cfg.dataloader, ChatDataLoaderConfig) and cfg.dataloader.data_files == "a.parquet"
    assert isinstance(cfg.dataloader.chat_encoder, DSV4EncoderConfig) and cfg.dataloader.chat_encoder.mode == "thinking"
    with pytest.raises(SystemExit):
        ConfigManager().parse_args(["--module", "llama3", "--config", "llama3_debugmodel", "dataloader:no_such_loader"])


def test_example_scripts_parse_with_the_real_config_parser(tmp_path):
    """Every example launcher runs through the launch scripts with the validator in place of the trainer."""
    import glob
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    assets = tmp_path / "hf"
    assets.mkdir()
    (assets / "tokenizer.json").write_text("{}")
    env = dict(os.environ, TRAIN_FILE="titan_b200.config.validate", COMM_MODE="fake_backend", NGPU="8",
               HF_ASSETS_PATH=str(assets), HF_CKPT=str(assets), DATA_FILES="x.parquet", NODE_RANK="0", NNODES="1",
               PYTHONPATH=root)
    scripts = sorted(glob.glob(os.path.join(root, "examples", "*", "*.sh")))
    assert len(scripts) >= 10
    from concurrent.futures import ThreadPoolExecutor

    def run(sh):   # the scripts are independent: a few at a time (each child spends seconds importing torch)
        return sh, subprocess.run(["bash", sh], env=env, capture_output=True, text=True, cwd=str(tmp_path))

    with ThreadPoolExecutor(max_workers=4) as pool:
        for sh, out in pool.map(run, scripts):
            assert out.returncode == 0, f"{sh}:\n{out.stdout[-2000:]}\n{out.stderr[-2000:]}"
            assert '"_type": "TrainerConfig"' in out.stdout, sh
