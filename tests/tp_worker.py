"""One tensor-parallel rank (a process with one GPU) for tests/test_tp_gpu.py.

usage: python tests/tp_worker.py RANK WORLD WORKDIR [int batch] [int new_tokens] [float16|int8]
Rank 0 creates the NCCL id and leaves it in WORKDIR/id.bin; every rank builds its shard of the TINY model, generates
greedily, and writes WORKDIR/out_<rank>.npz (ids, local logits slice, vocabulary offset).
"""
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from denograd_b200 import Device, synth  # noqa: E402
from denograd_b200.llama3 import Llama3  # noqa: E402
from denograd_b200.multi import TensorParallel  # noqa: E402
from tests.golden.gen_golden import TINY  # noqa: E402


def main() -> None:
    import faulthandler
    # a rank that stops making progress (its peer died, say) reports where it is and leaves by itself
    faulthandler.dump_traceback_later(90, exit=True)
    rank, world, work = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
    batch = int(sys.argv[4]) if len(sys.argv) > 4 else 2
    n_new = int(sys.argv[5]) if len(sys.argv) > 5 else 8
    quant = sys.argv[6] if len(sys.argv) > 6 else "float16"
    dev = Device[f"CUDA:{rank}"]
    id_path = os.path.join(work, "id.bin")
    if rank == 0:
        uid = TensorParallel.unique_id()
        with open(id_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(id_path + ".tmp", id_path)
    else:
        deadline = time.time() + 120
        while not os.path.exists(id_path):  # host-side wait with a deadline; no GPU work is pending meanwhile
            if time.time() > deadline:
                raise TimeoutError("rank 0 never published the NCCL id")
            time.sleep(0.05)
        uid = open(id_path, "rb").read()
    tp = TensorParallel(dev, rank, world, uid)
    if os.environ.get("JG_TP_PEER", "1") != "0":
        from denograd_b200.multi import exchange_via_directory
        ok = tp.open_peers(exchange_via_directory(work, rank, world))
        with open(os.path.join(work, f"peer_{rank}.txt"), "w") as f:
            f.write("1" if ok else "0")
    if quant == "missing-peer":
        missing_peer(dev, tp, rank, work)
        return
    arch = TINY
    if os.environ.get("JG_TEST_ARCH") == "step":  # a shape the single-kernel step takes under tensor parallelism
        from tests.util import TP_STEP_ARCH
        arch = TP_STEP_ARCH
    llm = Llama3(size="1B", args=arch, quantize=quant, max_context=64, max_batch=batch, tied_output=True, temperature=0, device=f"CUDA:{rank}", tp=tp).load_synthetic()
    prompt = synth.prompt_tokens(6, arch["vocab_size"], batch=batch, seed=31)
    ids = llm.generate(prompt, n_new)
    with open(os.path.join(work, f"step_{rank}.txt"), "w") as f:
        f.write("1" if llm.model._single_kernel_step(batch) is not None else "0")
    logits = llm.model.last_logits(batch)
    # the graph-replayed device loop must agree with the per-token API under sharding too
    llm2 = Llama3(size="1B", args=arch, quantize=quant, max_context=64, max_batch=batch, tied_output=True, temperature=0, device=f"CUDA:{rank}", tp=tp).load_synthetic()
    first = llm2._prefill(prompt).numpy()
    loop = llm2.model.decode_loop(first, llm2.start_pos, n_new - 1)
    np.savez(os.path.join(work, f"out_{rank}.npz"), ids=ids, logits=logits, offset=llm.model.vocab_offset,
             loop=np.concatenate([first[:, None], loop], axis=1))
    dev.synchronize()
    # the communicator is left to process exit: NCCL waits in ncclCommDestroy for captured graphs that still hold its
    # collectives, and the models (with their graphs) are alive here


def missing_peer(dev, tp, rank: int, work: str) -> None:
    """Failure detection without a GPU fault: both ranks do one exchange, then rank 0 starts a second one that rank 1
    never joins (rank 1 has nothing in flight and simply stops launching).  Rank 0's kernel gives up after the
    configured limit and records it; the next synchronising call reports JG_ETIMEDOUT and the device stays usable."""
    from denograd_b200 import ffi
    from denograd_b200.device import Tensor
    n = 4096
    part = Tensor(np.full((n,), float(rank + 1), np.float32), device=dev)
    h = Tensor(np.zeros((n,), np.float16), device=dev)
    ffi.call("jg_peer_allreduce_residual", tp.handle, h.ptr, part.ptr, n)  # both ranks: 1 + 2 = 3
    dev.synchronize()
    ok_first = bool((h.numpy() == 3).all())
    status, usable = 0, False
    if rank == 0:
        ffi.call("jg_peer_allreduce_residual", tp.handle, h.ptr, part.ptr, n)  # nobody answers
        try:
            dev.synchronize()
        except ffi.JgError as e:
            status = e.status
        # the context is intact: an ordinary kernel still runs and synchronises cleanly
        z = Tensor(np.ones((8,), np.float16), device=dev)
        dev.call("jg_fill_const_f16", z.ptr, 8, 2.0)
        dev.synchronize()
        usable = bool((z.numpy() == 2).all())
        with open(os.path.join(work, "rank0_done"), "w") as f:  # nothing of rank 0 addresses rank 1's memory any more
            f.write("1")
    else:
        # rank 1 has nothing in flight and launches nothing more, but it stays alive — its exchange buffer is mapped
        # into rank 0, whose abandoned exchange still stores into it — until rank 0 is through (host-side wait, bounded)
        deadline = time.time() + 60
        while not os.path.exists(os.path.join(work, "rank0_done")) and time.time() < deadline:
            time.sleep(0.05)
    np.savez(os.path.join(work, f"out_{rank}.npz"), ok_first=ok_first, status=status, usable=usable)


if __name__ == "__main__":
    main()
