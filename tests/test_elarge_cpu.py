"""eLargeModel: config normalisation / validation, YAML round trip, CLI actions, building a model + trainer."""

import json

import torch
import yaml

from easydel_b200.elarge import eLargeModel, normalize_config, validate_config
from easydel_b200.elarge.__main__ import main as cli

TINY = dict(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4,
            num_key_value_heads=2, max_position_embeddings=64)


def _cfg(tmp_path):
    return {"model": {"model_type": "llama"}, "base_config": {"values": TINY},
            "loader": {"dtype": "fp32", "param_dtype": "fp32"},
            "trainer": {"trainer_type": "sft", "max_training_steps": 2, "total_batch_size": 2, "learning_rate": 1e-3,
                        "save_directory": str(tmp_path), "do_last_save": False, "use_wandb": False,
                        "progress_bar_type": "none", "model_name": "t"}}


def test_normalize_and_validate():
    n = normalize_config({"model": "some/path"})
    assert n["model"]["name_or_path"] == "some/path" and n["esurge"]["page_size"] == 128
    assert n["sharding"]["axis_names"] == ["dp", "fsdp", "ep", "tp", "sp"]
    assert validate_config({"model": "x"}) == []
    bad = validate_config({"model": "x", "sharding": {"axis_dims": [-1, -1, 1, 1, 1]}, "loader": {"dtype": "fp64"},
                           "quantization": {"method": "int3"}, "trainer": {"trainer_type": "nope"}, "oops": {}})
    assert len(bad) == 5


def test_yaml_roundtrip_and_cli(tmp_path, capsys):
    e = eLargeModel(_cfg(tmp_path)).set_esurge(max_num_seqs=8).set_sharding([1, 1, 1, 1, 1])
    p = tmp_path / "cfg.yaml"
    e.to_yaml(str(p))
    again = eLargeModel.from_yaml(str(p))
    assert again.to_dict() == e.to_dict()
    assert cli([str(p)]) == 0 and "config OK" in capsys.readouterr().out
    assert cli([str(p), "--action", "to_json", "--set", "esurge.max_num_seqs=4"]) == 0
    assert json.loads(capsys.readouterr().out)["esurge"]["max_num_seqs"] == 4
    raw = yaml.safe_load(p.read_text())
    raw["esurge"]["bogus"] = 1
    p.write_text(yaml.safe_dump(raw))
    assert cli([str(p), "--action", "validate"]) == 1


def test_build_model_trainer_and_train(tmp_path):
    e = eLargeModel(_cfg(tmp_path))
    model = e.build_model()
    assert sum(p.numel() for p in model.parameters()) > 0 and model.dtype == torch.float32
    g = torch.Generator().manual_seed(0)
    data = [{"input_ids": torch.randint(3, 64, (16,), generator=g).tolist()} for _ in range(8)]
    for d in data:
        d["labels"] = d["input_ids"]
    out = e.train(train_dataset=data)
    assert out.state.step == 2
    eng = e.set_esurge(max_model_len=128, max_num_seqs=2).build_esurge()
    res = eng.generate([3, 4, 5], None)
    assert len(res[0].outputs[0].token_ids) > 0


def test_cluster_config_generator(tmp_path):
    import importlib.util
    import pathlib

    import yaml

    path = pathlib.Path(__file__).resolve().parents[1] / "autoscale" / "generate_cluster_configs.py"
    spec = importlib.util.spec_from_file_location("generate_cluster_configs", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    files = mod.generate("sft", 4, "img", "missing.yaml", "train", tmp_path)
    ray = yaml.safe_load(files["ray"].read_text())
    assert ray["max_workers"] == 3 and ray["available_node_types"]["b200_worker"]["resources"]["GPU"] == 8
    docs = list(yaml.safe_load_all(files["k8s"].read_text()))
    sts = [d for d in docs if d["kind"] == "StatefulSet"][0]
    assert sts["spec"]["replicas"] == 4
    args = sts["spec"]["template"]["spec"]["containers"][0]["args"][0]
    assert "--nnodes=4" in args and "--nproc-per-node=8" in args and "--master-addr=sft-0.sft" in args
    assert "#SBATCH --nodes=4" in files["slurm"].read_text()
