"""Expert-parallel parity on 2, 4 or 8 GPUs: the multi-rank worker that tests/test_ep_multi_gpu.py
launches under torchrun (pytest does not collect this file itself). By hand:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port 29511 tests/ep_multi_gpu.py [nccl|peer|peer_unfused|peer_mb2|peer_mb4|bench] [small|full]

(peer: the owner's DSD stores its rows into the source ranks' buffers from its epilogue;
peer_unfused: DSD writes y and a second kernel pushes it; peer_nodispatch: all rows are pushed by a kernel of
their own and every rank waits for all of them before the owner's routing; peer_mbM: the step cut into M micro-batches
pipelined over M streams; bench: exactly what the benchmark runs at this rank count.)

small: T=512 tokens per rank, D=256, F=512, E=32. Every rank builds the same global batch from a seed,
keeps its T tokens and its E/N experts.
full:  the benchmark's expert-parallel workload as the benchmark builds it: E=128, D=F=2048, T=4096
tokens per rank, permuted-Zipf routing, per-rank token seeds over shared weights, capacity T*k.

Either way a rank runs one expert-parallel step eagerly and one through a CUDA graph with fresh tokens
and routing, and checks its own rows against the fp32 oracle on its tokens with ALL experts
(rtol = atol = 2e-2) and the owner's layout against the single-process layout of the concatenated
batch. Prints one line per rank and exits non-zero on any mismatch.
"""

from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))

from oracle import layout as L  # noqa: E402
from oracle import moe as M  # noqa: E402
from sparsebench_b200.ep import ExpertParallelMoE, shard_experts  # noqa: E402
from sparsebench_b200.workloads import CONFIGS, _weights, make_layer, routing_case  # noqa: E402

T, D, F, E, K = 512, 256, 512, 32, 2


def global_batch(world: int, seed: int, case: str):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(world * T, D, generator=g).bfloat16()
    gate = torch.rand(world * T, K, generator=g).bfloat16()
    idx = routing_case(case, world * T, E, seed=seed)
    return x, idx, gate


def check_layout(layer, rank: int, world: int, idx: torch.Tensor, tokens: int = T, experts: int = E,
                 ffn_dim: int = F) -> None:
    """idx: the concatenated batch's expert_idx [world*tokens, k] (global token id = rank*tokens + t)."""
    trace = layer.last
    global_token = torch.where(trace.send_index >= 0, trace.send_index + rank * tokens, -1).to(torch.int32)
    received = torch.empty_like(global_token)
    dist.all_to_all_single(received, global_token)
    whole = L.build_topology(idx, experts, ffn_dim, 128)
    owner = trace.owner_layout
    per_rank = experts // world
    counts, offs = owner.tokens_per_expert.cpu().numpy(), owner.padded_offsets.cpu().numpy()
    rows, recv_np = owner.row_token.cpu().numpy(), received.cpu().numpy()
    for e_local in range(per_rank):
        e = rank * per_rank + e_local
        count = int(whole.tokens_per_expert[e])
        assert int(counts[e_local]) == count, f"expert {e}: {counts[e_local]} copies, expected {count}"
        got = recv_np[rows[offs[e_local] : offs[e_local] + count]]
        start = int(whole.padded_offsets[e])
        assert np.array_equal(got, whole.row_token[start : start + count]), f"expert {e}: copy order differs"


def finish(rank: int, world: int, local: int, layer, what: str) -> None:
    from sparsebench_b200 import _C

    assert int(_C.device_status(torch.device("cuda", local)).item()) == 0
    layer.check()
    print(f"rank {rank}/{world}: expert-parallel parity ok, {what}", flush=True)
    # Hard exit after a last barrier: destroying the communicator while a captured graph still holds
    # its collectives has been seen to block forever.
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


def main_full(rank: int, world: int, local: int, mode: str) -> None:
    """The benchmark's workload at the benchmark's size, set up the way the benchmark sets it up."""
    import bench_ep

    cfg = CONFIGS["expert_parallel"]
    tokens, k, experts = cfg.num_tokens, cfg.k, cfg.num_experts
    per_rank = experts // world
    mine = range(rank * per_rank, (rank + 1) * per_rank)
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // world))
    # All experts on the host for the oracle (per-expert seeds: identical on every rank); this rank's on its GPU.
    w1_all = _weights(0, range(experts), cfg.d_model, cfg.ffn_dim, 0, torch.bfloat16)
    w2_all = _weights(1, range(experts), cfg.ffn_dim, cfg.d_model, 0, torch.bfloat16)
    overlapped = mode != "peer_nodispatch"
    if mode == "bench":
        (overlapped, micro_batches), fuse, exchange = bench_ep.DEFAULT_EP_FORM.get(world, (False, 1)), True, "peer"
    elif mode == "bench_overlapped":
        micro_batches, fuse, exchange = 1, True, "peer"
    else:
        exchange = "peer" if mode.startswith("peer") else mode
        micro_batches = int(mode[len("peer_mb"):]) if mode.startswith("peer_mb") else 1
        fuse = mode != "peer_unfused"
    layer = ExpertParallelMoE(w1_all[mine.start:mine.stop].cuda(), w2_all[mine.start:mine.stop].cuda(), experts,
                              capacity=tokens * k, exchange=exchange, fuse_return=fuse, micro_batches=micro_batches,
                              fuse_dispatch=overlapped)

    def batch(shift: int):
        """Rank r's tokens as the benchmark draws them (token seed r + shift, weights and Zipf order seed 0)."""
        mine_in = make_layer(cfg, seed=0, token_seed=rank + shift, experts=range(0))  # tokens only, no weights
        everyone = torch.cat([routing_case(cfg.routing, tokens, experts, seed=r + shift, perm_seed=0) for r in range(world)])
        assert torch.equal(everyone[rank * tokens:(rank + 1) * tokens], mine_in.expert_idx)
        return mine_in, everyone

    def check(out: torch.Tensor, inputs, what: str) -> None:
        expected = M.moe_reference_streamed(inputs.x, inputs.expert_idx, inputs.expert_weight, w1_all, w2_all)
        err = (out.float().cpu() - expected).abs().max().item()
        torch.testing.assert_close(out.float().cpu(), expected, rtol=2e-2, atol=2e-2, msg=lambda m: f"{what}: {m}")
        print(f"rank {rank}: {what}: {tokens} rows within 2e-2 of the fp32 oracle (max abs err {err:.3e})", flush=True)

    inputs, everyone = batch(0)
    dx, didx, dgate = inputs.x.cuda(), inputs.expert_idx.cuda(), inputs.expert_weight.cuda()
    out = layer(dx, didx, dgate)
    torch.cuda.synchronize()
    layer.check()
    check(out, inputs, "eager")
    if layer.micro_batches == 1:
        check_layout(layer, rank, world, everyone, tokens, experts, cfg.ffn_dim)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        layer(dx, didx, dgate)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        graph_out = layer(dx, didx, dgate)
    inputs2, _ = batch(100)
    dx.copy_(inputs2.x.cuda())
    didx.copy_(inputs2.expert_idx.cuda())
    dgate.copy_(inputs2.expert_weight.cuda())
    graph.replay()
    torch.cuda.synchronize()
    check(graph_out, inputs2, "graph replay with new tokens and routing")
    finish(rank, world, local, layer, f"full size, exchange {mode}, micro-batches {layer.micro_batches}")


def main() -> None:
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if len(sys.argv) > 2 and sys.argv[2] == "full":
        main_full(rank, world, local, sys.argv[1])
        return
    g = torch.Generator().manual_seed(0)
    w1 = (torch.randn(E, D, F, generator=g) / D**0.5).bfloat16()
    w2 = (torch.randn(E, F, D, generator=g) / F**0.5).bfloat16()
    mode = sys.argv[1] if len(sys.argv) > 1 else "nccl"
    exchange = "peer" if mode.startswith("peer") else mode
    layer = ExpertParallelMoE(shard_experts(w1, rank, world).cuda(), shard_experts(w2, rank, world).cuda(), E,
                              capacity=T * K, exchange=exchange, fuse_return=mode != "peer_unfused",
                              fuse_dispatch=mode != "peer_nodispatch", push_beside=mode != "peer_warps",
                              micro_batches=2 if mode == "peer_split" else
                              int(mode[len("peer_mb"):]) if mode.startswith("peer_mb") else 1,
                              micro_fractions=(0.25, 0.75) if mode == "peer_split" else None)
    mine = slice(rank * T, (rank + 1) * T)

    def check(out: torch.Tensor, x, idx, gate, what: str) -> None:
        expected = M.moe_reference(x.float(), idx, gate.float(), w1.float(), w2.float())[mine]
        torch.testing.assert_close(out.float().cpu(), expected, rtol=2e-2, atol=2e-2, msg=lambda m: f"{what}: {m}")

    # Eager step.
    x, idx, gate = global_batch(world, 1, "zipf")
    dx, didx, dgate = x[mine].cuda(), idx[mine].cuda(), gate[mine].cuda()
    out = layer(dx, didx, dgate)
    torch.cuda.synchronize()
    layer.check()
    check(out, x, idx, gate, "eager")

    # Layout: the exchange keeps the stable global copy order (global token = rank*T + t).
    if layer.micro_batches == 1:  # with micro-batches each part has its own layout; the outputs cover those
        check_layout(layer, rank, world, idx)

    # Graph: capture once, replay with new tokens and routing.
    graph_ok = True
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            layer(dx, didx, dgate)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            graph_out = layer(dx, didx, dgate)
        x2, idx2, gate2 = global_batch(world, 2, "random")
        dx.copy_(x2[mine].cuda())
        didx.copy_(idx2[mine].cuda())
        dgate.copy_(gate2[mine].cuda())
        graph.replay()
        torch.cuda.synchronize()
        check(graph_out, x2, idx2, gate2, "graph replay")
    except AssertionError:
        raise
    except Exception as exc:  # capture of the collectives refused by this stack: report, do not hide
        graph_ok = False
        print(f"rank {rank}: graph capture unavailable: {exc!r}", flush=True)

    finish(rank, world, local, layer, f"exchange {mode} (graph replay {'ok' if graph_ok else 'not captured'})")


if __name__ == "__main__":
    main()
