"""The plain-torch distributed accretion backend (`coresets_b200.pytorch.accrete_distributed`) on a
two-rank gloo group against the lists the reference's own `accrete_distributed` produced
(tests/golden/torch_accrete.npz, keys `<case>_dist`; tests/golden/make_golden_torch_accrete.py)."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np

from tests.ports import address_in_use, free_port

ROOT = Path(__file__).resolve().parent.parent
WORKER = '''
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch, torch.distributed as dist
from coresets_b200.pytorch import accrete_distributed
from tests.golden.make_golden_torch_accrete import CASES, case_inputs, split_rows
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
torch.set_num_threads(1)
for name, c in CASES.items():
    Xa, Xc, order = case_inputs(c)
    out = accrete_distributed(split_rows(Xa, Xc, rank, world), order, Xa.shape[0], rank, world, max_k=c["max_k"], verbose=False)
    np.save(os.path.join({out!r}, f"{{name}}_{{rank}}.npy"), out.numpy())
dist.barrier()
dist.destroy_process_group()
'''


def test_distributed_torch_accrete_reproduces_the_reference(tmp_path):
    from tests.golden.make_golden_torch_accrete import CASES
    code = WORKER.format(root=str(ROOT), out=str(tmp_path))
    for attempt in range(3):
        port = free_port()
        procs = [subprocess.Popen([sys.executable, "-c", code],
                                  env=dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port)),
                                  stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for r in range(2)]
        outs = [p.communicate(timeout=600)[0] for p in procs]
        if any(p.returncode != 0 for p in procs) and address_in_use(outs) and attempt < 2:
            continue                                   # the rendezvous port was taken: another one
        break
    for r, p in enumerate(procs):
        assert p.returncode == 0, outs[r][-2000:]
    z = np.load(ROOT / "tests" / "golden" / "torch_accrete.npz")
    for name in CASES:
        for r in range(2):
            np.testing.assert_array_equal(np.load(tmp_path / f"{name}_{r}.npy"), z[name + "_dist"])
