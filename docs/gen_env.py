"""Regenerates docs/env.md from the parameter registry: python docs/gen_env.py (after make)."""
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
out = subprocess.run([os.path.join(ROOT, "nccl_b200", "bin", "ncclparam"), "--all"], capture_output=True, text=True, check=True).stdout
rows = []
for line in out.splitlines():
    if "=" not in line or "#" not in line:
        continue
    name, rest = line.split("=", 1)
    rows.append((name.strip(), rest.split("(")[0].strip(), rest.split("#", 1)[1].strip()))
with open(os.path.join(ROOT, "docs", "env.md"), "w") as f:
    f.write("# Environment variables\n\nGenerated from the parameter registry (`nccl_b200/bin/ncclparam --all`) by `docs/gen_env.py`. Variables shared with\n"
            "the reference keep its names and meaning; library-specific ones start with `NCCL_B200_`. Every variable can also be set\n"
            "in the configuration file named by `NCCL_CONF_FILE` (or `~/.nccl.conf`, `/etc/nccl.conf`) or by an environment plugin\n"
            "(`NCCL_ENV_PLUGIN`).\n\n| Variable | Default | Meaning |\n|---|---|---|\n")
    for n, v, d in rows:
        f.write("| `%s` | %s | %s |\n" % (n, ("`%s`" % v) if v else "(unset)", d.replace("|", "\\|")))
print("%d variables" % len(rows))
