"""A pretend Slurm for the tests: ``sbatch``, ``srun`` and ``scontrol`` that run everything on
this machine, at once, so the kit's job scripts run end to end without a cluster.

    python fake_slurm.py install DIR      writes DIR/{sbatch,srun,scontrol}

* ``sbatch [options] script``: reads ``#SBATCH`` lines and options (``--nodes``, ``--gres=gpu:N``,
  ``--job-name``, ``--output`` with ``%x``/``%j``, ``--parsable``), makes up ``SLURM_*``
  variables - every node is ``127.0.0.1``, so "the first node" is reachable - runs the script
  with bash and waits for it.  Prints the job id.  ``$FAKE_SLURM_LOG`` gets one line per call.
* ``srun [--ntasks=N] cmd``: N copies of ``cmd`` side by side, each with its ``SLURM_PROCID`` /
  ``SLURM_NODEID`` and a host name of its own (``GPUBRIDGE_SIM_HOSTNAME``), so ranks started
  by different tasks believe they sit on different boxes.  Exit code: the largest.
* ``scontrol show hostnames LIST``: one name per line.
"""
import os
import re
import subprocess
import sys


def log(line: str) -> None:
    path = os.environ.get("FAKE_SLURM_LOG")
    if path:
        with open(path, "a") as fh:
            fh.write(line + "\n")


def sbatch(argv: list[str]) -> int:
    options, script = {}, None
    for arg in argv:
        if arg.startswith("--"):
            key, _, value = arg[2:].partition("=")
            options[key] = value
        elif not arg.startswith("-"):
            script = arg
    if script is None or not os.path.isfile(script):
        print(f"fake sbatch: no job script in {argv}", file=sys.stderr)
        return 1
    declared = {}
    for line in open(script):
        found = re.match(r"#SBATCH\s+--([a-z-]+)(?:=(\S+))?", line)
        if found:
            declared[found.group(1)] = found.group(2) or ""
    merged = {**declared, **options}
    job = str(10000 + os.getpid() % 80000)
    nodes = int(merged.get("nodes", "1") or 1)
    name = merged.get("job-name") or os.path.basename(script)
    gres = merged.get("gres", "")
    env = dict(os.environ, SLURM_JOB_ID=job, SLURM_JOB_NAME=name, SLURM_NNODES=str(nodes),
               SLURM_JOB_NODELIST=",".join(["127.0.0.1"] * nodes), SLURM_SUBMIT_DIR=os.getcwd(),
               SLURM_GPUS_ON_NODE=gres.rpartition(":")[2] if gres.startswith("gpu:") else "0")
    log(f"sbatch {' '.join(argv)}")
    output = merged.get("output", "").replace("%x", name).replace("%j", job)
    if output:
        os.makedirs(os.path.dirname(os.path.abspath(output)), exist_ok=True)
        with open(output, "w") as fh:
            code = subprocess.run(["bash", script], env=env, stdout=fh, stderr=subprocess.STDOUT).returncode
    else:
        code = subprocess.run(["bash", script], env=env).returncode
    log(f"job {job} exit {code}")
    print(job if "parsable" in options else f"Submitted batch job {job}")
    return 0


def srun(argv: list[str]) -> int:
    tasks, rest = 1, list(argv)
    while rest and rest[0].startswith("-"):
        flag = rest.pop(0)
        if flag.startswith("--ntasks="):
            tasks = int(flag.partition("=")[2])
    log(f"srun x{tasks} {' '.join(rest[:4])}")
    children = []
    for task in range(tasks):
        env = dict(os.environ, SLURM_PROCID=str(task), SLURM_NODEID=str(task), SLURM_NTASKS=str(tasks),
                   GPUBRIDGE_SIM_HOSTNAME=f"fake-node-{task}")
        children.append(subprocess.Popen(rest, env=env))
    return max(child.wait() for child in children)


def scontrol(argv: list[str]) -> int:
    if argv[:2] != ["show", "hostnames"] or len(argv) != 3:
        print(f"fake scontrol: only 'show hostnames LIST', not {argv}", file=sys.stderr)
        return 1
    print("\n".join(argv[2].split(",")))
    return 0


def install(directory: str) -> None:
    os.makedirs(directory, exist_ok=True)
    for tool in ("sbatch", "srun", "scontrol"):
        path = os.path.join(directory, tool)
        with open(path, "w") as fh:
            fh.write(f'#!/usr/bin/env bash\nexec "{sys.executable}" "{os.path.abspath(__file__)}" {tool} "$@"\n')
        os.chmod(path, 0o755)


if __name__ == "__main__":
    tool, rest = sys.argv[1], sys.argv[2:]
    if tool == "install":
        install(rest[0])
        sys.exit(0)
    sys.exit({"sbatch": sbatch, "srun": srun, "scontrol": scontrol}[tool](rest))
