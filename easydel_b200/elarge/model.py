from __future__ import annotations

import copy
import json
import os
import typing as tp

import torch

# Sections and their defaults (easydel/infra/elarge/types/*.py, defaults.py). Unknown keys are rejected by
# ``validate_config`` so that typos in YAML files surface before a job is launched.
DEFAULTS: dict[str, dict] = {
    "model": {"name_or_path": None, "tokenizer": None, "task": "causal-language-model", "model_type": None,
              "extra_kwargs": {}},
    "loader": {"dtype": "bf16", "param_dtype": "bf16", "precision": None, "from_torch": None, "verbose": True,
               "trust_remote_code": False, "device": None},
    "sharding": {"axis_dims": [1, -1, 1, 1, 1], "axis_names": ["dp", "fsdp", "ep", "tp", "sp"], "dcn_axis_dims": None,
                 "auto_shard_model": True, "partition_rules": None},
    "quantization": {"method": None, "block_size": 64, "pattern": None, "quantize_tensors": True,
                     "kv_cache": None},
    "base_config": {"values": {}},
    "esurge": {"max_model_len": 8192, "max_num_seqs": 256, "max_num_batched_tokens": None, "hbm_utilization": 0.85,
               "page_size": 128, "enable_prefix_caching": True, "esurge_name": None, "tool_parser": None,
               "reasoning_parser": None, "host": "0.0.0.0", "port": 8000, "require_api_key": False,
               "admin_key": None, "sampling": {"max_tokens": 256, "temperature": 0.7, "top_p": 0.95}},
    "mixture": {"informs": [], "batch_size": 8, "seq_length": None, "pack": False, "pack_strategy": "first_fit",
                "seed": 0, "block_size": 64, "stop_strategy": "restart", "cache_dir": None},
    "eval": {"tasks": [], "num_fewshot": 0, "limit": None, "batch_size": 8, "max_new_tokens": 256,
             "output_path": None},
    "trainer": {"trainer_type": "sft"},   # every other key is passed to the trainer's arguments class
}
_FREE_FORM = {"trainer", "base_config", "model"}
_DTYPES = {"bf16": torch.bfloat16, "bfloat16": torch.bfloat16, "fp16": torch.float16, "float16": torch.float16,
           "fp32": torch.float32, "float32": torch.float32}


def normalize_config(cfg: dict | None) -> dict:
    """Fills every section with its defaults; ``model`` may be given as a bare string."""
    cfg = copy.deepcopy(cfg or {})
    if isinstance(cfg.get("model"), str):
        cfg["model"] = {"name_or_path": cfg["model"]}
    out = {}
    for sec, defaults in DEFAULTS.items():
        merged = copy.deepcopy(defaults)
        merged.update(cfg.get(sec) or {})
        out[sec] = merged
    for k, v in cfg.items():
        if k not in DEFAULTS:
            out[k] = v
    return out


def validate_config(cfg: dict) -> list[str]:
    """Returns a list of problems (empty when the config is usable)."""
    problems = []
    for k in cfg:
        if k not in DEFAULTS:
            problems.append(f"unknown section {k!r} (known: {sorted(DEFAULTS)})")
    for sec, defaults in DEFAULTS.items():
        if sec in _FREE_FORM:
            continue
        for k in (cfg.get(sec) or {}):
            if k not in defaults:
                problems.append(f"unknown key {sec}.{k}")
    n = normalize_config(cfg)
    if n["loader"]["dtype"] not in _DTYPES or n["loader"]["param_dtype"] not in _DTYPES:
        problems.append(f"loader.dtype / param_dtype must be one of {sorted(_DTYPES)}")
    dims = n["sharding"]["axis_dims"]
    if len(dims) != len(n["sharding"]["axis_names"]):
        problems.append("sharding.axis_dims and sharding.axis_names differ in length")
    if sum(1 for d in dims if d == -1) > 1:
        problems.append("sharding.axis_dims may contain at most one -1")
    q = n["quantization"]["method"]
    if q not in (None, "int8", "nf4", "affine", "mxfp4", "nvfp4", "mxfp8", "nvfp8", "a8bit", "a4bit"):
        problems.append(f"unknown quantization.method {q!r}")
    if n["model"]["name_or_path"] is None and not n["base_config"]["values"]:
        problems.append("model.name_or_path is required (or base_config.values for a from-scratch model)")
    from ..trainers import get_trainer_class

    try:
        get_trainer_class(n["trainer"].get("trainer_type", "sft"))
    except Exception:
        problems.append(f"unknown trainer.trainer_type {n['trainer'].get('trainer_type')!r}")
    return problems


class eLargeModel:
    """Builder facade: ``eLargeModel(cfg).build_model()``, ``.train()``, ``.eval()``, ``.build_esurge()``, ``.serve()``."""

    def __init__(self, config: dict | str | None = None, **sections):
        if isinstance(config, str):
            config = self._read(config)
        cfg = dict(config or {})
        cfg.update(sections)
        self.config = normalize_config(cfg)
        self._model = None
        self._tokenizer = None

    # ---- construction / serialisation -------------------------------------------------------------------
    @staticmethod
    def _read(path: str) -> dict:
        with open(path) as f:
            if path.endswith((".yaml", ".yml")):
                import yaml

                return yaml.safe_load(f) or {}
            return json.load(f)

    @classmethod
    def from_json(cls, path: str) -> "eLargeModel":
        return cls(cls._read(path))

    from_yaml = from_json

    @classmethod
    def from_pretrained(cls, name_or_path: str, **sections) -> "eLargeModel":
        return cls({"model": {"name_or_path": name_or_path}}, **sections)

    def to_dict(self) -> dict:
        return copy.deepcopy(self.config)

    def to_json(self, path: str | None = None) -> str:
        s = json.dumps(self.config, indent=2, default=str)
        if path:
            tmp = path + ".tmp"
            with open(tmp, "w") as f:
                f.write(s)
            os.replace(tmp, path)
        return s

    def to_yaml(self, path: str | None = None) -> str:
        import yaml

        s = yaml.safe_dump(json.loads(json.dumps(self.config, default=str)), sort_keys=False)
        if path:
            tmp = path + ".tmp"
            with open(tmp, "w") as f:
                f.write(s)
            os.replace(tmp, path)
        return s

    def validate(self) -> list[str]:
        return validate_config(self.config)

    # ---- fluent setters (the reference's ``set_*`` / ``update_*`` helpers) ---------------------------------
    def update(self, section: str, **kw) -> "eLargeModel":
        self.config.setdefault(section, {}).update(kw)
        return self

    def set_model(self, name_or_path: str) -> "eLargeModel":
        return self.update("model", name_or_path=name_or_path)

    def set_dtype(self, dtype: str, param_dtype: str | None = None) -> "eLargeModel":
        return self.update("loader", dtype=dtype, param_dtype=param_dtype or dtype)

    def set_sharding(self, axis_dims: tp.Sequence[int], axis_names: tp.Sequence[str] | None = None) -> "eLargeModel":
        kw = {"axis_dims": list(axis_dims)}
        if axis_names:
            kw["axis_names"] = list(axis_names)
        return self.update("sharding", **kw)

    def set_quantization(self, method: str | None, **kw) -> "eLargeModel":
        return self.update("quantization", method=method, **kw)

    def set_esurge(self, **kw) -> "eLargeModel":
        return self.update("esurge", **kw)

    def set_trainer(self, trainer_type: str, **kw) -> "eLargeModel":
        return self.update("trainer", trainer_type=trainer_type, **kw)

    def set_mixture(self, informs: list[dict], **kw) -> "eLargeModel":
        return self.update("mixture", informs=informs, **kw)

    def add_dataset(self, data_files, type: str | None = None, content_field: str = "text", weight: float = 1.0,  # noqa: A002
                    **kw) -> "eLargeModel":
        """Appends one source to ``mixture.informs`` (fluent form of the YAML list)."""
        informs = list(self.config["mixture"].get("informs") or [])
        informs.append(dict(data_files=data_files, type=type, content_field=content_field, weight=weight, **kw))
        return self.update("mixture", informs=informs)

    def set_eval(self, tasks: list[str], **kw) -> "eLargeModel":
        return self.update("eval", tasks=tasks, **kw)

    # ---- builders ---------------------------------------------------------------------------------------------
    def model_kwargs(self) -> dict:
        """Keyword arguments for ``AutoEasyDeLModel*.from_pretrained`` (builders.py:87)."""
        c = self.config
        kw = dict(dtype=_DTYPES[c["loader"]["dtype"]], param_dtype=_DTYPES[c["loader"]["param_dtype"]],
                  sharding_axis_dims=tuple(c["sharding"]["axis_dims"]),
                  sharding_axis_names=tuple(c["sharding"]["axis_names"]),
                  auto_shard_model=c["sharding"]["auto_shard_model"], config_kwargs=dict(c["base_config"]["values"]),
                  from_torch=c["loader"]["from_torch"], device=c["loader"]["device"], verbose=c["loader"]["verbose"])
        if c["quantization"]["method"]:
            from ..layers.quantization import EasyDeLQuantizationConfig

            kw["quantization_config"] = EasyDeLQuantizationConfig(dtype=c["quantization"]["method"],
                                                                  block_size=c["quantization"]["block_size"],
                                                                  pattern=c["quantization"]["pattern"])
            kw["apply_quantization"] = True
        kw.update(c["model"].get("extra_kwargs") or {})
        return kw

    def build_tokenizer(self):
        if self._tokenizer is None:
            from transformers import AutoTokenizer

            path = self.config["model"]["tokenizer"] or self.config["model"]["name_or_path"]
            self._tokenizer = AutoTokenizer.from_pretrained(path)
            if self._tokenizer.pad_token_id is None:
                self._tokenizer.pad_token = self._tokenizer.eos_token
        return self._tokenizer

    def build_model(self):
        if self._model is not None:
            return self._model
        from ..infra.factory import TaskType, registry
        from ..modules.auto import auto_modeling as A

        c = self.config
        task = TaskType(c["model"]["task"])
        path = c["model"]["name_or_path"]
        if path is None:
            mtype = c["model"]["model_type"] or "llama"
            cfg = registry.get_config(mtype)(sharding_axis_dims=tuple(c["sharding"]["axis_dims"]),
                                             **c["base_config"]["values"])
            reg = registry.get_module_registration(task, mtype)
            self._model = reg.module.sequential_init(cfg, dtype=_DTYPES[c["loader"]["dtype"]],
                                                     param_dtype=_DTYPES[c["loader"]["param_dtype"]],
                                                     device=c["loader"]["device"])
            return self._model
        cls = A.resolve_model_class(path, task)
        self._model = cls.from_pretrained(path, **self.model_kwargs())
        return self._model

    def build_dataset(self, tokenizer=None):
        """``mixture.informs`` -> a packed / mixed source (builders.py: mixture + tokenized dataset)."""
        from ..data import DatasetConfig, Pipeline, PipelineConfig

        m = self.config["mixture"]
        if not m["informs"]:
            return None
        ds = [DatasetConfig(data_files=i["data_files"], type=i.get("type"), name=i.get("name"),
                            content_field=i.get("content_field", "text"), messages_field=i.get("messages_field"),
                            weight=i.get("weight", 1.0), columns=i.get("columns")) for i in m["informs"]]
        pc = PipelineConfig(datasets=ds, seq_length=m["seq_length"], pack=m["pack"], pack_strategy=m["pack_strategy"],
                            batch_size=m["batch_size"], seed=m["seed"], mixture_block_size=m["block_size"],
                            stop_strategy=m["stop_strategy"], cache_dir=m["cache_dir"])
        return Pipeline.from_config(pc, tokenizer).build()

    def build_training_arguments(self):
        from ..trainers import get_trainer_arguments_class

        t = dict(self.config["trainer"])
        ttype = t.pop("trainer_type", "sft")
        cls = get_trainer_arguments_class(ttype)
        import dataclasses

        known = {f.name for f in dataclasses.fields(cls)}
        unknown = sorted(k for k in t if k not in known)
        if unknown:
            raise ValueError(f"unknown trainer arguments for {ttype!r}: {unknown}")
        return cls(**t)

    def build_trainer(self, train_dataset=None, eval_dataset=None, **extra):
        from ..trainers import get_trainer_class

        ttype = self.config["trainer"].get("trainer_type", "sft")
        model = self.build_model()
        tok = extra.pop("processing_class", None)
        if tok is None and (self.config["model"]["tokenizer"] or self.config["model"]["name_or_path"]):
            try:
                tok = self.build_tokenizer()
            except Exception:
                tok = None
        if train_dataset is None:
            train_dataset = self.build_dataset(tok)
        args = self.build_training_arguments()
        cls = get_trainer_class(ttype)
        try:
            return cls(arguments=args, model=model, processing_class=tok, train_dataset=train_dataset,
                       eval_dataset=eval_dataset, **extra)
        except TypeError:
            return cls(arguments=args, model=model, dataset_train=train_dataset, dataset_eval=eval_dataset, **extra)

    def train(self, **kw):
        return self.build_trainer(**kw).train()

    def build_esurge(self, tokenizer=None):
        from ..inference.esurge import eSurge

        e = self.config["esurge"]
        tok = tokenizer
        if tok is None:
            try:
                tok = self.build_tokenizer()
            except Exception:
                tok = None
        return eSurge(self.build_model(), tokenizer=tok, max_model_len=e["max_model_len"],
                      max_num_seqs=e["max_num_seqs"], max_num_batched_tokens=e["max_num_batched_tokens"],
                      hbm_utilization=e["hbm_utilization"], page_size=e["page_size"],
                      enable_prefix_caching=e["enable_prefix_caching"], esurge_name=e["esurge_name"])

    def build_server(self, tokenizer=None):
        from ..inference.esurge.server import eSurgeApiServer

        e = self.config["esurge"]
        return eSurgeApiServer(self.build_esurge(tokenizer), require_api_key=e["require_api_key"],
                               admin_key=e["admin_key"], tool_parser=e["tool_parser"],
                               reasoning_parser=e["reasoning_parser"],
                               default_max_tokens=e["sampling"].get("max_tokens", 256))

    def serve(self, tokenizer=None):
        e = self.config["esurge"]
        self.build_server(tokenizer).run(host=e["host"], port=e["port"])

    def eval(self, tokenizer=None) -> dict:
        """Runs the configured lm-eval tasks through the eSurge adapter (benchmarking.py:40-615)."""
        from ..inference.evaluations import eSurgeLMEvalAdapter, run_lm_eval

        ev = self.config["eval"]
        adapter = eSurgeLMEvalAdapter(self.build_esurge(tokenizer), max_new_tokens=ev["max_new_tokens"],
                                      batch_size=ev["batch_size"])
        res = run_lm_eval(adapter, ev["tasks"], num_fewshot=ev["num_fewshot"], limit=ev["limit"])
        if ev["output_path"]:
            with open(ev["output_path"], "w") as f:
                json.dump(res, f, indent=2, default=str)
        return res

    def run_benchmarks(self, tasks: list[str] | None = None, tokenizer=None, **kw) -> dict:
        """lm-eval tasks through the serving engine; ``tasks`` / keyword overrides replace the ``eval`` section's."""
        if tasks is not None or kw:
            self.update("eval", **({"tasks": tasks} if tasks is not None else {}), **kw)
        return self.eval(tokenizer)

    def __repr__(self):
        m = self.config["model"]
        return f"eLargeModel(model={m['name_or_path']!r}, task={m['task']!r}, trainer={self.config['trainer'].get('trainer_type')!r})"
