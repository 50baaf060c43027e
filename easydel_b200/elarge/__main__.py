"""YAML / JSON runner (easydel/scripts/elarge.py):

    python -m easydel_b200.elarge CONFIG.yaml [--action validate|train|eval|serve|print|dump_config|to_json|to_yaml]
                                              [--out PATH] [--set section.key=value ...]

The action defaults to the config's top-level ``action`` key, else ``validate``.
"""

from __future__ import annotations

import argparse
import json
import sys

from .model import eLargeModel

ACTIONS = ("validate", "train", "eval", "serve", "print", "dump_config", "to_json", "to_yaml")


def _coerce(v: str):
    try:
        return json.loads(v)
    except json.JSONDecodeError:
        return v


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m easydel_b200.elarge")
    ap.add_argument("config")
    ap.add_argument("--action", choices=ACTIONS, default=None)
    ap.add_argument("--out", default=None)
    ap.add_argument("--set", action="append", default=[], metavar="section.key=value")
    args = ap.parse_args(argv)
    raw = eLargeModel._read(args.config)
    action = args.action or raw.pop("action", None) or "validate"
    raw.pop("action", None)
    for item in args.set:
        path, _, val = item.partition("=")
        sec, _, key = path.partition(".")
        raw.setdefault(sec, {})[key] = _coerce(val)
    elm = eLargeModel(raw)
    problems = elm.validate()
    if action == "validate":
        for p in problems:
            print("error:", p)
        print("config OK" if not problems else f"{len(problems)} problem(s)")
        return 1 if problems else 0
    if action in ("print", "dump_config", "to_json"):
        print(elm.to_json(args.out))
        return 0
    if action == "to_yaml":
        print(elm.to_yaml(args.out))
        return 0
    if problems:
        for p in problems:
            print("error:", p, file=sys.stderr)
        return 1
    if action == "train":
        out = elm.train()
        print(json.dumps({"final_step": out.state.step, "checkpoint": out.checkpoint_path}))
    elif action == "eval":
        print(json.dumps(elm.eval(), indent=2, default=str))
    elif action == "serve":
        elm.serve()
    return 0


if __name__ == "__main__":
    sys.exit(main())
