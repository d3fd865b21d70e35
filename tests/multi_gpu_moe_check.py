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
    T, H, I, k, E = 384, 512, 256, 4, 3      # 1536 routed pairs per rank: above the scheduler's 1024-thread stride
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
    # ---- the same forward cut into minibatches on three streams: same bytes everywhere
    cb_first = cb.clone()
    dist.barrier()
    cb.fill_(-3.0)
    torch.cuda.synchronize()
    dist.barrier()
    outs2 = mx8.dispatch_mlp_swiglu_combine_fwd(x, x_ptrs, cb, cb_ptrs, None, wgq.to(dev), wgs.to(dev), None, wuq.to(dev),
                                                wus.to(dev), None, wdq.to(dev), wds.to(dev), pr, pt, nt, tpe, k, 28, 0, 512)
    assert mx8.device_status() == 0
    torch.cuda.synchronize()
    dist.barrier()
    assert torch.equal(cb.view(torch.int16), cb_first.view(torch.int16)), "pipelined forward: combine buffer differs"
    assert torch.equal(outs2[12][:n].view(torch.int16), outs[12][:n].view(torch.int16)), "pipelined forward: y_routed differs"
    assert torch.equal(outs2[0][:, :n].view(torch.uint8), outs[0][:, :n].view(torch.uint8)), "pipelined forward: x_fp8_t differs"
    assert torch.equal(outs2[9][:, :n].view(torch.uint8), outs[9][:, :n].view(torch.uint8)), "pipelined forward: hidden_fp8_t differs"
    # ---- backward over peer memory: prologue, barrier, fused backward, barrier, epilogue
    def weights_T(r):
        wg = torch.stack([O.make_input(I, H, seed=100 + 10 * r + e, std=H ** -0.5) for e in range(E)])
        wu = torch.stack([O.make_input(I, H, seed=200 + 10 * r + e, std=H ** -0.5) for e in range(E)])
        wd = torch.stack([O.make_input(H, I, seed=300 + 10 * r + e, std=I ** -0.5) for e in range(E)])
        return [O.quantize_both(w.transpose(1, 2).contiguous())[:2] for w in (wg, wu, wd)]

    bw = weights_T(rank)
    d_out_all = torch.stack([O.make_input(T, H, seed=400 + r, std=H ** -0.5) for r in range(world)])
    d_cb = symm_mem.empty(T * k, H, dtype=torch.bfloat16, device=dev)
    d_cb_ptrs = list(symm_mem.rendezvous(d_cb, group).buffer_ptrs)
    d_xb = symm_mem.empty(T * k, H, dtype=torch.bfloat16, device=dev)
    d_xb.zero_()
    d_xb_ptrs = list(symm_mem.rendezvous(d_xb, group).buffer_ptrs)
    mx8.bwd_prologue(d_out_all[rank].to(dev), w_all[rank].to(dev), d_cb)
    torch.cuda.synchronize()
    dist.barrier()
    dv = lambda pair: (pair[0].to(dev), pair[1].to(dev))
    b = mx8.dispatch_mlp_swiglu_combine_bwd(None, d_cb, d_cb_ptrs, d_xb, d_xb_ptrs, None, *dv(bw[0]), None, *dv(bw[1]), None, *dv(bw[2]),
                                            outs[0], outs[1], None, outs[3], outs[4], None, outs[6], outs[7], None, outs[9], outs[10],
                                            x, x_ptrs, wgq.to(dev), wgs.to(dev), wuq.to(dev), wus.to(dev), pr, pt, nt, tpe, k)
    assert mx8.device_status() == 0
    torch.cuda.synchronize()
    dist.barrier()
    d_x = mx8.bwd_epilogue_routed(None, d_xb, k)
    torch.cuda.synchronize()
    d_cb_refs = [MO.bwd_prologue_ref(d_out_all[r], w_all[r]) for r in range(world)]
    bwd_refs = []
    for r in range(world):
        m = refs[r]["y"].shape[0]
        d_y = torch.zeros(m, H, dtype=torch.bfloat16)
        for src in range(world):
            sel = prs[r][:m] == src
            d_y[sel] = d_cb_refs[src][pts[r][:m][sel].long()]
        rtpe = MO.schedule_ref(ids_all_cpu, E, cap, r)[3]
        bwd_refs.append(MO.expert_mlp_bwd_ref(d_y, refs[r], rtpe, *weights_T(r)))
    assert torch.equal(b[10][:n].view(torch.uint8).cpu(), bwd_refs[rank]["d_y_fp8"]), "gathered gradient rows differ"
    for idx, key in ((13, "d_w_gate"), (15, "d_w_up"), (17, "d_w_down")):
        rel = O.rel_frobenius(b[idx].cpu(), bwd_refs[rank][key])
        assert rel < 2e-2, (key, rel)
    dxb_ref = MO.combine_ref([r["d_x"] for r in bwd_refs], prs, pts, rank, T, k)
    rel_dx = O.rel_frobenius(d_x.cpu(), MO.bwd_epilogue_ref(None, dxb_ref, k))
    assert rel_dx < 2e-2, rel_dx
    # ---- the same backward in minibatches on three streams: same bytes in every rank's gradient buffer
    d_xb_first = d_xb.clone()
    dist.barrier()
    d_xb.fill_(-3.0)
    torch.cuda.synchronize()
    dist.barrier()
    b2 = mx8.dispatch_mlp_swiglu_combine_bwd(None, d_cb, d_cb_ptrs, d_xb, d_xb_ptrs, None, *dv(bw[0]), None, *dv(bw[1]), None, *dv(bw[2]),
                                             outs[0], outs[1], None, outs[3], outs[4], None, outs[6], outs[7], None, outs[9], outs[10],
                                             x, x_ptrs, wgq.to(dev), wgs.to(dev), wuq.to(dev), wus.to(dev), pr, pt, nt, tpe, k, 28, 0, 512)
    assert mx8.device_status() == 0
    torch.cuda.synchronize()
    dist.barrier()
    assert torch.equal(d_xb.view(torch.int16), d_xb_first.view(torch.int16)), "pipelined backward: gradient buffer differs"
    for idx in (13, 15, 17):
        assert torch.equal(b2[idx].view(torch.int16), b[idx].view(torch.int16)), "pipelined backward: weight gradient differs"
    flag = torch.ones(1, device=dev)
    dist.all_reduce(flag)
    if rank == 0:
        print(f"MULTI_GPU_MOE_OK world={world} rel_y={rel_y:.2e} rel_out={rel_out:.2e} rel_dx={rel_dx:.2e}", flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
