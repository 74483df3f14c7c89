"""Two-GPU runs of the tensor-parallel layer and the expert-parallel MoE block over NCCL (one process
per GPU).  Skipped on a single-GPU machine; the CPU suite covers the same bookkeeping with gloo."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, q):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        from arcquant_b200 import synth
        from arcquant_b200.llama_layer import (LlamaLayerConfig, QLlamaDecoderLayerTP, random_layer_weights,
                                               random_reorder_indices)
        from arcquant_b200.moe_block import MoEConfig, QMixtralMoEBlockEP, random_moe_weights, route_top_k

        dev = torch.device("cuda", rank)
        # --- tensor-parallel layer: the NCCL all-reduce must give what adding the partials by hand gives
        cfg = LlamaLayerConfig(hidden=1024, n_heads=8, n_kv_heads=4, head_dim=128, ffn=2048, select_num=64)
        W, I = random_layer_weights(cfg, 0), random_reorder_indices(cfg, 1)
        x = synth.activations(64, cfg.hidden, 4, synth.outlier_channels(cfg.hidden, 10, 3)).reshape(1, 64, -1).to(dev)
        pos = torch.arange(64, device=dev)
        y = QLlamaDecoderLayerTP(cfg, W, I, tp_rank=rank, tp_size=world, device=dev)(x, pos)
        ranks = [QLlamaDecoderLayerTP(cfg, W, I, tp_rank=r, tp_size=world, device=dev) for r in range(world)]
        x2 = x.reshape(64, -1)
        h = x2 + sum(r.attn_partial(x2, 1, 64, pos).float() for r in ranks).to(torch.bfloat16)
        ref = (h + sum(r.mlp_partial(h).float() for r in ranks).to(torch.bfloat16)).reshape(1, 64, -1)
        err_tp = float((y.float() - ref.float()).norm() / ref.float().norm())
        # the overlapped schedule (row chunks, asynchronous all-reduces) must give the same bytes
        x8 = synth.activations(512, cfg.hidden, 6, synth.outlier_channels(cfg.hidden, 10, 3)).reshape(1, 512, -1).to(dev)
        pos8 = torch.arange(512, device=dev)
        layer = QLlamaDecoderLayerTP(cfg, W, I, tp_rank=rank, tp_size=world, device=dev)
        y_plain = layer(x8, pos8)
        layer.overlap_rows = 128
        y_over = layer(x8, pos8)
        if not torch.equal(y_plain, y_over):
            err_tp = max(err_tp, 1.0)
        # sequence-parallel form: this rank's token shard in, the same rows of the output back
        rows_s = 512 // world
        y_sp = layer.forward_sequence_parallel(x8.reshape(512, -1)[rank * rows_s:(rank + 1) * rows_s].contiguous(), 1, 512, pos8)
        ref_sp = y_plain.reshape(512, -1)[rank * rows_s:(rank + 1) * rows_s]
        err_sp = float((y_sp.float() - ref_sp.float()).norm() / ref_sp.float().norm())
        if err_sp > 2e-3:      # (bit-equal with two ranks; a sum of more partials may be ordered differently)
            err_tp = max(err_tp, 1.0 + err_sp)
        # pipelined sequence-parallel form: 4 runs of one sequence, this rank's slice of every run
        xb = synth.activations(1024, cfg.hidden, 8, synth.outlier_channels(cfg.hidden, 10, 3)).reshape(4, 256, -1).to(dev)
        posb = torch.arange(256, device=dev)
        layer.overlap_rows = 1 << 30
        y_ref = layer(xb, posb).reshape(1024, -1)
        own = layer.pipelined_shard_rows(1024, world, rank, 4).to(dev)
        y_pp = layer.forward_sequence_parallel_pipelined(xb.reshape(1024, -1)[own].contiguous(), 4, 256, posb, 4)
        err_pp = float((y_pp.float() - y_ref[own].float()).norm() / y_ref[own].float().norm())
        if err_pp > 2e-3:
            err_tp = max(err_tp, 2.0 + err_pp)
        # the same with the row-parallel projections storing straight into the owners' memory
        layer.enable_peer_scatter(512)
        y_ps = layer.forward_sequence_parallel(x8.reshape(512, -1)[rank * rows_s:(rank + 1) * rows_s].contiguous(), 1, 512, pos8)
        y_ps2 = layer.forward_sequence_parallel(x8.reshape(512, -1)[rank * rows_s:(rank + 1) * rows_s].contiguous(), 1, 512, pos8)
        err_ps = float((y_ps.float() - ref_sp.float()).norm() / ref_sp.float().norm())
        if err_ps > 2e-3 or not torch.equal(y_ps, y_ps2):
            err_tp = max(err_tp, 3.0 + err_ps)
        dist.barrier()
        layer.disable_peer_scatter()
        # --- expert-parallel MoE block: same per-expert batches as one rank owning every expert
        mcfg = MoEConfig(hidden=1024, ffn=2048, n_experts=4, top_k=2, select_num=64)
        MW = random_moe_weights(mcfg, 0)
        xt = synth.activations(96, mcfg.hidden, 5, synth.outlier_channels(mcfg.hidden, 10, 3)).to(dev)
        ids, w = route_top_k(xt, MW["router"].to(dev), mcfg.top_k)
        full = QMixtralMoEBlockEP(mcfg, MW, device=dev)(xt, routing=(ids, w))
        lo, hi = rank * 96 // world, (rank + 1) * 96 // world
        part = QMixtralMoEBlockEP(mcfg, MW, ep_rank=rank, ep_size=world, device=dev)(
            xt[lo:hi].contiguous(), routing=(ids[lo:hi].contiguous(), w[lo:hi].contiguous()))
        err_ep = float((part.float() - full[lo:hi].float()).norm() / full[lo:hi].float().norm())
        # the same with rows stored straight into the peers' memory (twice: the buffers are reused)
        peer = QMixtralMoEBlockEP(mcfg, MW, ep_rank=rank, ep_size=world, device=dev)
        peer.enable_peer_dispatch(hi - lo, None)
        for _ in range(2):
            got = peer(xt[lo:hi].contiguous(), routing=(ids[lo:hi].contiguous(), w[lo:hi].contiguous()))
            if not torch.equal(got, full[lo:hi]) or peer.dispatcher.overflowed():
                err_ep = max(err_ep, 1.0)
        dist.barrier()
        peer.disable_peer_dispatch()
        q.put((rank, err_tp, err_ep))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tp_layer_and_ep_moe_over_nccl():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=120)
    for rank, err_tp, err_ep in res:
        assert err_tp < 1e-2, (rank, err_tp)      # bf16 all-reduce vs fp32 hand sum
        assert err_ep < 1e-2, (rank, err_ep)      # identical expert batches, different row grouping in transit
