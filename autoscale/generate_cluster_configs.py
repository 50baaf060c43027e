"""Cluster files for multi-node B200 jobs (the counterpart of the reference's Ray-on-TPU generator,
autoscale/generate-cluster-configs.py): from a node count and a job file it writes

* ``<name>-ray.yaml``      a Ray cluster description (head + GPU workers, 8 GPUs each) for the Ray trainer / data path,
* ``<name>-k8s.yaml``      a headless Service + indexed StatefulSet that starts ``torchrun`` on every node,
* ``<name>-slurm.sbatch``  the same launch under Slurm.

No cloud API is called: quotas and node pools are whatever the operator's cluster offers.

    python autoscale/generate_cluster_configs.py --name sft-70b --nodes 4 --job job.yaml --image easydel-b200
"""

from __future__ import annotations

import argparse
from pathlib import Path

import yaml

GPUS_PER_NODE = 8


def ray_config(name: str, nodes: int, image: str, gpus: int = GPUS_PER_NODE) -> dict:
    node = {"resources": {"CPU": 96, "GPU": gpus, "b200": gpus}, "node_config": {"image": image}}
    return {
        "cluster_name": name,
        "max_workers": max(nodes - 1, 0),
        "idle_timeout_minutes": 10,
        "docker": {"image": image, "container_name": "easydel", "run_options": ["--gpus=all", "--ipc=host",
                                                                             "--ulimit memlock=-1"]},
        "provider": {"type": "local", "head_ip": "${HEAD_IP}", "worker_ips": [f"${{WORKER_{i}_IP}}"
                                                                              for i in range(1, nodes)]},
        "available_node_types": {
            "head": dict(node, min_workers=0, max_workers=0),
            "b200_worker": dict(node, min_workers=max(nodes - 1, 0), max_workers=max(nodes - 1, 0)),
        },
        "head_node_type": "head",
        "head_start_ray_commands": ["ray stop", "ray start --head --port=6379 --dashboard-host=0.0.0.0"],
        "worker_start_ray_commands": ["ray stop", "ray start --address=$RAY_HEAD_IP:6379"],
    }


def _torchrun(nodes: int, gpus: int, rank: str, addr: str, job: str, action: str) -> list[str]:
    return ["python", "-m", "torch.distributed.run", f"--nnodes={nodes}", f"--node-rank={rank}",
            f"--nproc-per-node={gpus}", f"--master-addr={addr}", "--master-port=29500", "-m", "easydel_b200.elarge",
            job, "--action", action]


def k8s_manifests(name: str, nodes: int, image: str, job: str, action: str, gpus: int = GPUS_PER_NODE) -> list[dict]:
    svc = {"apiVersion": "v1", "kind": "Service", "metadata": {"name": name},
           "spec": {"clusterIP": "None", "selector": {"app": name}, "ports": [{"port": 29500, "name": "rdzv"}]}}
    cmd = _torchrun(nodes, gpus, "$(NODE_RANK)", f"{name}-0.{name}", "/config/job.yaml", action)
    pod = {
        "metadata": {"labels": {"app": name}},
        "spec": {
            "restartPolicy": "Always",
            "containers": [{
                "name": "trainer", "image": image, "command": ["bash", "-c"],
                "args": ["export NODE_RANK=${HOSTNAME##*-}; exec " + " ".join(cmd).replace("$(NODE_RANK)",
                                                                                          "$NODE_RANK")],
                "resources": {"limits": {"nvidia.com/gpu": gpus}},
                "volumeMounts": [{"name": "job", "mountPath": "/config"}, {"name": "shm", "mountPath": "/dev/shm"}],
                "env": [{"name": "NCCL_DEBUG", "value": "WARN"}],
            }],
            "volumes": [{"name": "job", "configMap": {"name": f"{name}-job"}},
                        {"name": "shm", "emptyDir": {"medium": "Memory"}}],
        },
    }
    sts = {"apiVersion": "apps/v1", "kind": "StatefulSet", "metadata": {"name": name},
           "spec": {"serviceName": name, "replicas": nodes, "podManagementPolicy": "Parallel",
                    "selector": {"matchLabels": {"app": name}}, "template": pod}}
    cm = {"apiVersion": "v1", "kind": "ConfigMap", "metadata": {"name": f"{name}-job"},
          "data": {"job.yaml": Path(job).read_text() if Path(job).exists() else "# put the eLargeModel config here\n"}}
    return [svc, cm, sts]


def slurm_script(name: str, nodes: int, job: str, action: str, gpus: int = GPUS_PER_NODE) -> str:
    cmd = " ".join(_torchrun(nodes, gpus, "$SLURM_NODEID", "$MASTER_ADDR", job, action))
    return (f"#!/bin/bash\n#SBATCH --job-name={name}\n#SBATCH --nodes={nodes}\n#SBATCH --ntasks-per-node=1\n"
            f"#SBATCH --gpus-per-node={gpus}\n#SBATCH --exclusive\n"
            "export MASTER_ADDR=$(scontrol show hostnames $SLURM_JOB_NODELIST | head -n 1)\n"
            f"srun bash -c '{cmd}'\n")


def generate(name: str, nodes: int, image: str, job: str, action: str, out_dir: str | Path,
             gpus: int = GPUS_PER_NODE) -> dict[str, Path]:
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    files = {"ray": out / f"{name}-ray.yaml", "k8s": out / f"{name}-k8s.yaml", "slurm": out / f"{name}-slurm.sbatch"}
    files["ray"].write_text(yaml.safe_dump(ray_config(name, nodes, image, gpus), sort_keys=False))
    files["k8s"].write_text(yaml.safe_dump_all(k8s_manifests(name, nodes, image, job, action, gpus), sort_keys=False))
    files["slurm"].write_text(slurm_script(name, nodes, job, action, gpus))
    return files


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__.split("\n")[0])
    ap.add_argument("--name", default="easydel-b200")
    ap.add_argument("--nodes", type=int, default=1)
    ap.add_argument("--gpus-per-node", type=int, default=GPUS_PER_NODE)
    ap.add_argument("--image", default="easydel-b200")
    ap.add_argument("--job", default="job.yaml")
    ap.add_argument("--action", default="train", choices=["train", "serve", "eval"])
    ap.add_argument("--output-dir", default=str(Path(__file__).parent / "generated"))
    ap.add_argument("--print-summary", action="store_true")
    a = ap.parse_args(argv)
    files = generate(a.name, a.nodes, a.image, a.job, a.action, a.output_dir, a.gpus_per_node)
    if a.print_summary:
        print(f"{a.nodes} node(s) x {a.gpus_per_node} B200 = {a.nodes * a.gpus_per_node} ranks")
    for k, p in files.items():
        print(f"{k}: {p}")


if __name__ == "__main__":
    main()
