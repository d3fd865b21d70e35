"""Two or more ranks, one GPU each: the MoE forward over peer-mapped (symmetric) memory against the
CPU oracle.  Launched by tests/test_gpu_multi.py through torchrun; prints MULTI_GPU_MOE_OK on rank 0."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "gpu-experiments_b200"))

import mx8  # noqa: E402
from oracle import moe_oracle as MO  # noqa: E402
from oracle import mx8_oracle as O  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    import torch.distributed._symmetric_memory as symm_mem
    group = dist.group.WORLD.group_name
    if hasattr(symm_mem, "enable_symm_mem_for_group"):
        try:
            symm_mem.enable_symm_mem_for_group(group)
        except Exception:
            pass
    T, H, I, k, E = 256, 512, 256, 4, 3
    cap = ((world * T * k) // 256 + E) * 256
    g = torch.Generator().manual_seed(7)
    logits = torch.randn(world * T, world * E, generator=g)
    ids_all_cpu, w_all = MO.route(logits, k)
    ids_all_cpu, w_all = ids_all_cpu.view(world, T, k), w_all.view(world, T, k)
    x_all = torch.stack([O.make_input(T, H, seed=90 + r) for r in range(world)])

    x = symm_mem.empty(T, H, dtype=torch.bfloat16, device=dev)
    x.copy_(x_all[rank])
    x_ptrs = list(symm_mem.rendezvous(x, group).buffer_ptrs)
    cb = symm_mem.empty(T * k, H, dtype=torch.bfloat16, device=dev)
    cb.zero_()
    cb_ptrs = list(symm_mem.rendezvous(cb, group).buffer_ptrs)

    def weights(r):
        wg = torch.stack([O.make_input(I, H, seed=100 + 10 * r + e, std=H ** -0.5) for e in range(E)])
        wu = torch.stack([O.make_input(I, H, seed=200 + 10 * r + e, std=H ** -0.5) for e in range(E)])
        wd = torch.stack([O.make_input(H, I, seed=300 + 10 * r + e, std=I ** -0.5) for e in range(E)])
        return [O.quantize_both(w)[:2] for w in (wg, wu, wd)]

    (wgq, wgs), (wuq, wus), (wdq, wds) = weights(rank)
    ids = ids_all_cpu[rank].to(dev)
    ids_all = torch.empty(world, T, k, dtype=torch.int32, device=dev)
    torch.cuda.synchronize()
    dist.barrier()

    dist.all_gather_into_tensor(ids_all, ids)
    pr, pt, nt, tpe = mx8.schedule(ids_all, E, cap, rank)
    outs = mx8.dispatch_mlp_swiglu_combine_fwd(x, x_ptrs, cb, cb_ptrs, None, wgq.to(dev), wgs.to(dev), None, wuq.to(dev),
                                               wus.to(dev), None, wdq.to(dev), wds.to(dev), pr, pt, nt, tpe, k)
    assert mx8.device_status() == 0
    torch.cuda.synchronize()
    dist.barrier()                                     # every rank's pushes have landed
    out = mx8.fwd_epilogue(None, cb, w_all[rank].to(dev))
    torch.cuda.synchronize()

    # ---- oracle for every rank (small), then compare this rank's share
    assert torch.equal(ids_all.cpu(), ids_all_cpu)
    refs, prs, pts = [], [], []
    for r in range(world):
        rpr, rpt, rnt, rtpe, _ = MO.schedule_ref(ids_all_cpu, E, cap, r)
        n = int(rnt)
        refs.append(MO.expert_mlp_ref(MO.dispatch_ref(x_all, rpr, rpt, n, k), rtpe, *weights(r)))
        prs.append(rpr)
        pts.append(rpt)
    n = int(nt)
    assert torch.equal(pr.cpu(), prs[rank]) and int(nt) == refs[rank]["y"].shape[0]
    assert torch.equal(outs[0][:, :n].view(torch.uint8).cpu(), refs[rank]["x_fp8_t"]), "dispatched + quantized tokens differ"
    rel_y = O.rel_frobenius(outs[12][:n].cpu(), refs[rank]["y"])
    assert rel_y < 1e-2, rel_y
    cb_ref = MO.combine_ref([r["y"] for r in refs], prs, pts, rank, T, k)
    ref_out = MO.fwd_epilogue_ref(torch.zeros(T, H, dtype=torch.bfloat16), cb_ref, w_all[rank])
    rel_out = O.rel_frobenius(out.cpu(), ref_out)
    assert rel_out < 1e-2, rel_out
    # exactness of the data movement: the combine buffer holds exactly the rows the experts produced
    ys = [torch.empty(cap, H, dtype=torch.bfloat16, device=dev) for _ in range(world)]
    dist.all_gather(ys, outs[12].contiguous())
    nts = [torch.empty(1, dtype=torch.int32, device=dev) for _ in range(world)]
    dist.all_gather(nts, nt)
    cb_own = MO.combine_ref([ys[r][:int(nts[r])].cpu() for r in range(world)], prs, pts, rank, T, k)
    touched = torch.zeros(T * k, dtype=torch.bool)
    for r in range(world):
        m = int(nts[r])
        sel = prs[r][:m] == rank
        touched[pts[r][:m][sel].long()] = True
    assert bool(touched.all())
    assert torch.equal(cb.cpu().view(torch.int16), cb_own.view(torch.int16)), "combine buffer differs from the expert outputs"
    flag = torch.ones(1, device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print(f"MULTI_GPU_MOE_OK world={world} rel_y={rel_y:.2e} rel_out={rel_out:.2e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
