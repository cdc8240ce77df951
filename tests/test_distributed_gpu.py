"""One process per GPU over NCCL: collectives, the FFN with a split contracted
dim and the MoE layer with its alltoalls, each rank against the oracle.
Skipped when fewer than two GPUs are visible."""

import os
import socket

import numpy as np
import pytest

from mesh_b200 import mtf
from helpers import rel_err, rng

pytestmark = pytest.mark.gpu


def _free_port():
  s = socket.socket()
  s.bind(("127.0.0.1", 0))
  port = s.getsockname()[1]
  s.close()
  return port


def _worker(rank, world, port, out_dir):
  import torch
  import torch.distributed as dist
  from mesh_b200.cuda_mesh_impl import CudaMeshImpl
  from oracle.numpy_mesh_impl import NumpyMeshImpl
  from oracle.numpy_ops import Arr
  os.environ["MASTER_ADDR"] = "127.0.0.1"
  os.environ["MASTER_PORT"] = str(port)
  torch.cuda.set_device(rank)
  dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
  try:
    mesh_shape = "all:%d" % world
    impl = CudaMeshImpl(mesh_shape, "d_ff:all", list(range(world)))
    assert impl.is_distributed and impl.local_pnums == [rank]
    ora = NumpyMeshImpl(mesh_shape, "d_ff:all")
    ops = impl.slice_ops
    r = rng(1)
    vals = [r.standard_normal((4, 8, 6)).astype(np.float32) for _ in range(world)]
    a = ora.LaidOutTensor([Arr(v.copy(), mtf.float32) for v in vals])
    b = impl.LaidOutTensor([ops.from_host(vals[rank], mtf.float32)])

    def check(x, y, exact=True):
      p, q = x.tensor_list[rank].a, ops.to_host(y.tensor_list[0])
      assert p.shape == q.shape
      if exact:
        np.testing.assert_array_equal(p, q)
      else:
        assert rel_err(q, p) < 1e-6
    for name in ("SUM", "MAX", "MIN"):
      check(ora.allreduce(a, [0], name), impl.allreduce(b, [0], name), exact=(name != "SUM"))
    for ca in range(3):
      check(ora.allconcat(a, 0, ca), impl.allconcat(b, 0, ca))
      for sa in range(3):
        if vals[0].shape[sa] % world == 0:
          check(ora.alltoall(a, 0, sa, ca), impl.alltoall(b, 0, sa, ca))
    for offset, wrap in ((1, False), (-1, True)):
      check(ora.shift_by_n_processors(a, 0, offset, wrap), impl.shift_by_n_processors(b, 0, offset, wrap))

    # the alltoall as one kernel over peer memory (mtfc_alltoall_peer): every (split,
    # concat) pair, three calls in a row on the same buffers and flags, a bf16 tensor of
    # the MoE layer's shape, and a recorded call replayed
    nat_a2a = __import__("mesh_b200._native", fromlist=["x"])
    peer = CudaMeshImpl(mesh_shape, "d_ff:all", list(range(world)))
    peer.PEER_ALLTOALL_MIN_BYTES = 1
    big = [r.standard_normal((8, 16, 128)).astype(np.float32) for _ in range(world)]
    a2 = ora.LaidOutTensor([Arr(v.copy(), mtf.float32) for v in big])
    b2 = peer.LaidOutTensor([ops.from_host(big[rank], mtf.float32)])
    for sa in range(3):
      for ca in range(3):
        want = ora.alltoall(a2, 0, sa, ca)
        for _ in range(3):
          check(want, peer.alltoall(b2, 0, sa, ca))
    from oracle.numpy_ops import round_to_bf16
    routed = [round_to_bf16(r.standard_normal((2, 8, 4, 6, 64)).astype(np.float32)) for _ in range(world)]
    a3 = ora.LaidOutTensor([Arr(v.copy(), mtf.bfloat16) for v in routed])
    b3 = peer.LaidOutTensor([ops.from_host(routed[rank], mtf.bfloat16)])
    check(ora.alltoall(a3, 0, 1, 2), peer.alltoall(b3, 0, 1, 2))
    check(ora.alltoall(a3, 0, 2, 1), peer.alltoall(b3, 0, 2, 1))
    used = list(getattr(peer, "_a2a_ws", {}).values())
    assert len(used) >= 2 and all(w is not None for w in used), "the peer-memory alltoall did not run"
    want = ora.alltoall(a2, 0, 1, 0)
    res, run = peer.capture(lambda: peer.alltoall(b2, 0, 1, 0))
    for _ in range(3):
      run()
      check(want, res)
    nat_a2a.device_status()   # raises if a bounded wait ran out
    peer.release_graphs()
    # results live in slots of the peer-mapped buffer: more live results than slots (the
    # extra ones are copies of the shared slot) all stay intact, and the slots come back
    # when the results are dropped
    ws_big = [w for (_, nbytes), w in peer._a2a_ws.items() if nbytes == big[0].nbytes][0]
    import gc
    res = run = None
    gc.collect()
    free_before = len(ws_big.free)
    assert free_before == peer.PEER_ALLTOALL_SLOTS
    held = [peer.alltoall(b2, 0, 1, 0) for _ in range(free_before + 2)]
    assert len(ws_big.free) == 0
    for h in held:
      check(want, h)
    del held, h
    gc.collect()
    assert len(ws_big.free) == free_before

    def ffn(backend):
      rr = rng(2)
      g = mtf.Graph()
      m = mtf.Mesh(g, "m")
      x = rr.standard_normal((4, 64, 128)).astype(np.float32)
      wi = (rr.standard_normal((128, 512)) / 11).astype(np.float32)
      wo = (rr.standard_normal((512, 128)) / 22).astype(np.float32)
      X = mtf.import_tf_tensor(m, x, "batch:4,length:64,d_model:128", dtype=mtf.bfloat16)
      WI = mtf.import_tf_tensor(m, wi, "d_model:128,d_ff:512", dtype=mtf.bfloat16)
      WO = mtf.import_tf_tensor(m, wo, "d_ff:512,d_model:128", dtype=mtf.bfloat16)
      y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", 512), wi=WI, wo=WO)
      low = mtf.Lowering(g, {m: backend})
      return low.export_to_tf_tensor(y), low.counter_totals()
    got, cg = ffn(impl)
    ref, cr = ffn(ora)
    assert rel_err(got, ref) < 2e-2 and cg == cr and "allreduce/[0]/einsum_op" in cg
    # the same with the contraction cut in chunks whose allreduces overlap it
    eager = CudaMeshImpl(mesh_shape, "d_ff:all", list(range(world)))
    eager.OVERLAP_MIN_ROWS = 1
    launches = __import__("mesh_b200._native", fromlist=["x"]).launch_count()
    got2, cg2 = ffn(eager)
    assert __import__("mesh_b200._native", fromlist=["x"]).launch_count() - launches >= 1 + eager.OVERLAP_CHUNKS
    assert rel_err(got2, ref) < 2e-2 and cg2 == cr

    # the same with the contraction and its allreduce as ONE kernel over peer memory
    # (mtfc_gemm_allreduce): three lowerings on the same buffers (the flag epochs
    # advance), then the recorded lowering replayed as a CUDA graph
    def ffn_big(backend, replay=False):
      rr = rng(3)
      g = mtf.Graph()
      m = mtf.Mesh(g, "m")
      x = rr.standard_normal((8, 150, 128)).astype(np.float32)
      wi = (rr.standard_normal((128, 512)) / 11).astype(np.float32)
      wo = (rr.standard_normal((512, 128)) / 22).astype(np.float32)
      X = mtf.import_tf_tensor(m, x, "batch:8,length:150,d_model:128", dtype=mtf.bfloat16)
      WI = mtf.import_tf_tensor(m, wi, "d_model:128,d_ff:512", dtype=mtf.bfloat16)
      WO = mtf.import_tf_tensor(m, wo, "d_ff:512,d_model:128", dtype=mtf.bfloat16)
      y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", 512), wi=WI, wo=WO)
      if not replay:
        return mtf.Lowering(g, {m: backend}).export_to_tf_tensor(y)
      res, run = backend.capture(lambda: mtf.Lowering(g, {m: backend}).tensors[y].to_laid_out_tensor())
      outs = []
      for _ in range(3):
        run()
        outs.append(ops.to_host(res.tensor_list[0]))
      return outs
    ref_big = ffn_big(ora)
    nat_mod = __import__("mesh_b200._native", fromlist=["x"])
    import torch
    exchange = []
    # every exchange form: remote epilogue stores, peer loads by the owner, and the
    # switch's multicast addresses (multimem) where the fabric offers them
    for form in ("push", "pull", "multimem"):
      fused = CudaMeshImpl(mesh_shape, "d_ff:all", list(range(world)))
      fused.OVERLAP_MIN_ROWS = 1
      fused.PIPELINED_ALLREDUCE = False
      fused.FUSED_ALLREDUCE = True
      fused.FUSED_MIN_BYTES = 1
      fused.FUSED_EXCHANGE = form
      for _ in range(3):
        before = nat_mod.launch_count()
        got_big = ffn_big(fused)
        used = nat_mod.launch_count() - before
        assert rel_err(got_big, ref_big) < 2e-2
      ws = [w for w in getattr(fused, "_peer_ws", {}).values()]
      assert ws and all(w is not None for w in ws), "the fused einsum+allreduce path did not run"
      exchange.append({0: "push", 1: "pull", 2: "multimem"}[ws[0].exchange])
      assert used < 1 + fused.OVERLAP_CHUNKS + 4   # one launch for the contraction, not one per chunk
      nat_mod.device_status()   # raises if a bounded wait ran out
      for o in ffn_big(fused, replay=True):
        assert rel_err(o, ref_big) < 2e-2
      # every rank holds the same bits
      mine = torch.from_numpy(np.ascontiguousarray(got_big).view(np.int32).astype(np.int64)).cuda().sum().reshape(1)
      hi, lo = mine.clone(), mine.clone()
      dist.all_reduce(hi, op=dist.ReduceOp.MAX)
      dist.all_reduce(lo, op=dist.ReduceOp.MIN)
      assert int(hi.item()) == int(lo.item())
      fused.release_graphs()

    # the row-split schedule of x.wi -> ReLU -> .wo (the first product stays pending and the
    # contraction + allreduce takes both over): weight slices gathered, every rank multiplies
    # its share of the rows with the whole hidden dim, row blocks gathered chunk by chunk
    def ffn_wide(backend, replay=False):
      rr = rng(5)
      g = mtf.Graph()
      m = mtf.Mesh(g, "m")
      x = rr.standard_normal((8, 512, 256)).astype(np.float32)
      wi = (rr.standard_normal((256, 1024)) / 16).astype(np.float32)
      wo = (rr.standard_normal((1024, 256)) / 32).astype(np.float32)
      X = mtf.import_tf_tensor(m, x, "batch:8,length:512,d_model:256", dtype=mtf.bfloat16)
      WI = mtf.import_tf_tensor(m, wi, "d_model:256,d_ff:1024", dtype=mtf.bfloat16)
      WO = mtf.import_tf_tensor(m, wo, "d_ff:1024,d_model:256", dtype=mtf.bfloat16)
      y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", 1024), wi=WI, wo=WO)
      if not replay:
        low = mtf.Lowering(g, {m: backend})
        return low.export_to_tf_tensor(y), low.counter_totals()
      res, run = backend.capture(lambda: mtf.Lowering(g, {m: backend}).tensors[y].to_laid_out_tensor())
      outs = []
      for _ in range(3):
        run()
        outs.append(ops.to_host(res.tensor_list[0]))
      return outs
    split = CudaMeshImpl(mesh_shape, "d_ff:all", list(range(world)))
    split.RESHARDED_FFN_MIN_BYTES = 1
    split.RESHARDED_FFN_MIN_CHUNK_ROWS = 256
    ref_wide, counters_wide = ffn_wide(ora)
    for _ in range(3):
      got_wide, counters_got = ffn_wide(split)
      assert rel_err(got_wide, ref_wide) < 2e-2 and counters_got == counters_wide
    ws = list(getattr(split, "_ffn_ws", {}).values())
    assert ws and all(w is not None for w in ws), "the row-split FFN schedule did not run"
    nat_mod.device_status()
    for o in ffn_wide(split, replay=True):
      assert rel_err(o, ref_wide) < 2e-2
    mine = torch.from_numpy(np.ascontiguousarray(got_wide).view(np.int32).astype(np.int64)).cuda().sum().reshape(1)
    hi, lo = mine.clone(), mine.clone()
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    assert int(hi.item()) == int(lo.item())    # every rank holds the same bits
    split.release_graphs()
    exchange.append("row-split x%d chunks" % list(split._ffn_ws)[0][-1])
    # the other chunking (little to move beside the arithmetic: two chunks, the last a quarter)
    split2 = CudaMeshImpl(mesh_shape, "d_ff:all", list(range(world)))
    split2.RESHARDED_FFN_MIN_BYTES = 1
    split2.RESHARDED_FFN_MIN_CHUNK_ROWS = 256
    split2.RESHARDED_FFN_LINK_BYTES_PER_S = 1e15
    for _ in range(2):
      got_wide2, _ = ffn_wide(split2)
      assert rel_err(got_wide2, ref_wide) < 2e-2
    assert list(split2._ffn_ws)[0][-1] == 2 and all(w is not None for w in split2._ffn_ws.values())
    nat_mod.device_status()
    # the reference's schedule stays available
    plain = CudaMeshImpl(mesh_shape, "d_ff:all", list(range(world)))
    plain.RESHARDED_FFN = False
    got_plain, _ = ffn_wide(plain)
    assert rel_err(got_plain, ref_wide) < 2e-2 and not getattr(plain, "_ffn_ws", {})

    # the pipelined form: un-chunked GEMM with progress counters, exchange by the copy
    # engines on a second stream; eager three times (the counters' epochs advance),
    # then recorded once and replayed
    def ffn_rows(backend, replay=False):
      rr = rng(4)
      g = mtf.Graph()
      m = mtf.Mesh(g, "m")
      x = rr.standard_normal((8, 256, 128)).astype(np.float32)
      wi = (rr.standard_normal((128, 512)) / 11).astype(np.float32)
      wo = (rr.standard_normal((512, 128)) / 22).astype(np.float32)
      X = mtf.import_tf_tensor(m, x, "batch:8,length:256,d_model:128", dtype=mtf.bfloat16)
      WI = mtf.import_tf_tensor(m, wi, "d_model:128,d_ff:512", dtype=mtf.bfloat16)
      WO = mtf.import_tf_tensor(m, wo, "d_ff:512,d_model:128", dtype=mtf.bfloat16)
      y = mtf.layers.dense_relu_dense(X, mtf.Dimension("d_ff", 512), wi=WI, wo=WO)
      if not replay:
        return mtf.Lowering(g, {m: backend}).export_to_tf_tensor(y)
      res, run = backend.capture(lambda: mtf.Lowering(g, {m: backend}).tensors[y].to_laid_out_tensor())
      outs = []
      for _ in range(3):
        run()
        outs.append(ops.to_host(res.tensor_list[0]))
      return outs
    piped = CudaMeshImpl(mesh_shape, "d_ff:all", list(range(world)))
    piped.OVERLAP_MIN_ROWS = 1
    piped.PIPELINED_ALLREDUCE = True
    piped.PIPELINE_MIN_BYTES = 1
    piped.FUSED_ALLREDUCE = False
    ref_rows = ffn_rows(ora)
    for _ in range(3):
      got_rows = ffn_rows(piped)
      assert rel_err(got_rows, ref_rows) < 2e-2
    ws = [w for w in getattr(piped, "_pipe_ws", {}).values()]
    assert ws and all(w is not None for w in ws), "the pipelined einsum+allreduce path did not run"
    nat_mod.device_status()
    for o in ffn_rows(piped, replay=True):
      assert rel_err(o, ref_rows) < 2e-2
    mine = torch.from_numpy(np.ascontiguousarray(got_rows).view(np.int32).astype(np.int64)).cuda().sum().reshape(1)
    hi, lo = mine.clone(), mine.clone()
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    assert int(hi.item()) == int(lo.item())    # every rank holds the same bits
    piped.release_graphs()
    exchange.append("pipelined x%d chunks" % ws[0].chunks)

    layout = "batch:all;experts:all"

    def moe(backend):
      rr = rng(6)
      g = mtf.Graph()
      m = mtf.Mesh(g, "m")
      bb, l, d, f, e = 8, 64, 64, 128, 8
      x = rr.standard_normal((bb, l, d)).astype(np.float32)
      wg = (rr.standard_normal((d, e)) / 8).astype(np.float32)
      wi = (rr.standard_normal((e, d, f)) / 8).astype(np.float32)
      wo = (rr.standard_normal((e, f, d)) / 11).astype(np.float32)
      X = mtf.import_tf_tensor(m, x, "batch:8,length:64,d_model:64", dtype=mtf.bfloat16)
      WG = mtf.import_tf_tensor(m, wg, "d_model:64,expert_unsplit:8", dtype=mtf.float32)
      WI = mtf.import_tf_tensor(m, wi, "experts:8,d_model:64,d_ff:128", dtype=mtf.bfloat16)
      WO = mtf.import_tf_tensor(m, wo, "experts:8,d_ff:128,d_model:64", dtype=mtf.bfloat16)
      hp = mtf.moe.HParams(moe_group_size=64, moe_second_policy_train="all")
      out, loss, aux = mtf.moe.transformer_moe_layer_v1(
          X, mtf.Dimension("d_model", d), hp, True, mesh_shape, layout, WG, WI, WO, return_aux=True)
      low = mtf.Lowering(g, {m: backend})
      return (low.export_to_tf_tensor(out), low.export_to_tf_tensor(aux["index_1"]),
              low.export_to_tf_tensor(aux["position_2"]), float(low.export_to_tf_tensor(loss)))
    go, gi, gp, gl = moe(CudaMeshImpl(mesh_shape, layout, list(range(world))))
    ro, ri, rp, rl = moe(NumpyMeshImpl(mesh_shape, layout))
    same = np.all(gi == ri, axis=-1)
    assert same.mean() > 0.8
    np.testing.assert_array_equal(gp[same], rp[same])
    assert rel_err(go.reshape(ri.shape + (-1,))[same], ro.reshape(ri.shape + (-1,))[same]) < 2e-2
    assert abs(gl - rl) < 2e-2 * abs(rl)
    impl.synchronize()
    open(os.path.join(out_dir, "ok%d" % rank), "w").write("ok exchange=%s cooperative=%d"
                                                       % (exchange, nat_mod.lib().mtfc_gemm_allreduce_cooperative()))
  finally:
    dist.destroy_process_group()


def test_one_process_per_gpu_over_nccl(tmp_path):
  import torch
  import torch.multiprocessing as mp
  world = min(torch.cuda.device_count(), 4)
  if world < 2:
    pytest.skip("needs at least two GPUs")
  world = 2 if world < 4 else 4
  mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
  assert sorted(os.listdir(str(tmp_path))) == ["ok%d" % r for r in range(world)]
  print(open(os.path.join(str(tmp_path), "ok0")).read())
