"""Worker of the tensor-parallel tests: run under torch.distributed.run, one process per GPU.
Compares the sharded decoder layer with the unsharded CPU oracle on this rank's block of rows."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "torch-spyre_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl")     # (no device_id: with spyre registered it is the accelerator type, not cuda)
    from oracle import llama_ref as L, math_ref
    from torch_spyre import _abi, stick_ops as K, tensor_parallel as TP

    d_model, heads, ffn, batch, seq = (int(v) for v in sys.argv[1:6])
    cfg = L.LayerConfig(d_model=d_model, heads=heads, ffn=ffn)
    if len(sys.argv) > 6:      # a whole model: vocabulary size and number of layers follow
        return model_case(rank, world, cfg, batch, seq, int(sys.argv[6]), int(sys.argv[7]))
    w = L.make_weights(cfg)
    x = torch.randn(batch, seq, d_model, generator=torch.Generator().manual_seed(0)).half()
    cos, sin = L.rope_tables(seq, cfg.head_dim)
    tp = TP.TPGroup()
    layer = TP.TPDecoderLayer(tp, w, heads, cfg.eps, cos, sin, batch, seq)
    rows = batch * seq // world
    mine = x.reshape(batch * seq, d_model)[rank * rows:(rank + 1) * rows].contiguous()
    xs = K.copy_host_to_sticks(mine.pin_memory())
    for _ in range(2):          # twice: the buffers are reused from call to call
        y = layer(xs)
    got = K.from_sticks(y).cpu()
    torch.cuda.synchronize()
    assert _abi.lib().ts_gemm_error_state() == 0 and _abi.lib().ts_attention_error_state() == 0
    cpu16 = L.layer_forward(x, w, cfg).reshape(batch * seq, d_model)[rank * rows:(rank + 1) * rows]
    truth = L.layer_forward_fp32(x, w, cfg).reshape(batch * seq, d_model)[rank * rows:(rank + 1) * rows]
    # the sharded sums add world partial products and the residual in fp16, in arrival order: a few more
    # roundings than the unsharded layer, so twice CPU fp16 eager's distance from the fp32 evaluation is allowed
    e = math_ref.assert_no_worse_than_cpu_fp16(got, cpu16, truth, factor=2.0, what=f"TP layer rank {rank}")
    ok = torch.tensor([1], device="cuda")
    dist.all_reduce(ok)
    if rank == 0:
        print(f"TP_OK world={world} nvlink_bytes_per_rank={layer.nvlink_bytes_per_call} "
              f"gpu_max={e['gpu_max']:.3e} cpu_max={e['cpu_max']:.3e} within_tol={e['frac_within_tol']:.4f}")
    dist.destroy_process_group()


def model_case(rank, world, cfg, batch, seq, vocab, n_layers):
    """Token ids -> logits through TPLlamaModel against the unsharded CPU oracle, on this rank's rows."""
    from oracle import llama_ref as L, math_ref
    from torch_spyre import _abi, stick_ops as K, tensor_parallel as TP

    mw = L.make_model_weights(cfg, vocab, n_layers)
    ids = torch.randint(0, vocab, (batch, seq), generator=torch.Generator().manual_seed(3))
    cos, sin = L.rope_tables(seq, cfg.head_dim)
    tp = TP.TPGroup()
    model = TP.TPLlamaModel(tp, mw, cfg.heads, cfg.eps, cos, sin, batch, seq)
    rows = batch * seq // world
    mine = ids.reshape(-1)[rank * rows:(rank + 1) * rows].contiguous().cuda()
    for _ in range(2):          # twice: the layers share one set of peer buffers, reused from call to call
        logits = model(mine)
    got = K.from_sticks(logits).cpu()
    torch.cuda.synchronize()
    lib = _abi.lib()
    assert lib.ts_gemm_error_state() == 0 and lib.ts_attention_error_state() == 0 and lib.ts_gather_error_state() == 0
    assert got.shape == (rows, vocab)
    cpu16 = L.model_forward(ids, mw, cfg).reshape(batch * seq, vocab)[rank * rows:(rank + 1) * rows]
    truth = L.model_forward(ids, mw, cfg, dtype=torch.float32).reshape(batch * seq, vocab)[rank * rows:(rank + 1) * rows]
    e = math_ref.assert_no_worse_than_cpu_fp16(got, cpu16, truth, factor=2.0, what=f"TP model rank {rank}")
    ok = torch.tensor([1], device="cuda")
    dist.all_reduce(ok)
    if rank == 0:
        print(f"TP_OK world={world} model layers={n_layers} gpu_max={e['gpu_max']:.3e} cpu_max={e['cpu_max']:.3e} "
              f"within_tol={e['frac_within_tol']:.4f}")
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
