"""Builds, through the reference's builder API, the tiled matrix product its authors sketch in
tmp/ir.mlir:1-17 (parallel grid, tiles in shared / local buffers, a k loop of two copies and a
gemm, a copy of the accumulator tile to C).  `tweak` lets a test break one aspect at a time."""
import frisk as F


def build_tiled_matmul(M, N, K, TM, TN, TK, dtype="fp16", accumulate=False, kstep=1, tweak=None,
                       row_reduce=None):
    """`row_reduce` = (kind, clear): after the accumulator tile is stored, reduce it over its columns
    into a [TM] buffer and copy that to a fourth kernel argument of M elements -- the gemm + reduce
    pair of the reference's attention sketch (tmp/ir.mlir:112-135) written as a tile program."""
    ctx = F.context()
    F.frisk.load_dialects(ctx)
    b = F.builder(ctx)
    module = b.create_module()
    module.context = ctx
    if tweak == "gemm_scaled":  # scales go with 8-bit float tiles only
        dtype = "e4m3fn"
    ty = {"fp16": b.get_f16_ty, "bf16": b.get_bf16_ty, "fp32": b.get_f32_ty,
          "e4m3fn": b.get_f8e4m3fn_ty}[dtype]()
    mk = lambda shape: b.get_memref_ty(ty, shape, F.AffineMap(), F.MemorySpace.GLOBAL)
    arg_tys = [mk([M, K]), mk([K, N]), mk([M, N])] + ([mk([M])] if row_reduce else [])
    kernel = b.create_kernel_op(module, "matmul", b.get_kernel_ty(arg_tys))
    module.push_back(kernel)
    entry = kernel.add_entry_block()
    b.set_insertion_point_to_start(entry)
    A, B, C = (entry.get_argument(i) for i in range(3))
    grid = [M // TM, N // TN]
    if tweak == "grid_short":
        grid[0] -= 1
    par = b.create_parallel_op(grid, 128)
    body = par.add_entry_block()
    b.set_insertion_point_to_start(body)
    by, bx = body.get_argument(0), body.get_argument(1)
    sA = b.create_alloc_buffer_op([TM, TK], dtype, F.MemorySpace.SHARED, 1024).get_result(0)
    sB = b.create_alloc_buffer_op([TK, TN], dtype, F.MemorySpace.SHARED, 1024).get_result(0)
    acc = b.create_alloc_buffer_op([TM, TN], dtype, F.MemorySpace.LOCAL).get_result(0)
    if tweak == "gemm_scaled":
        assert TM == TN
        sS = b.create_alloc_buffer_op([TM], "fp32", F.MemorySpace.SHARED).get_result(0)
    d0, d1 = b.get_affine_dim_expr(0), b.get_affine_dim_expr(1)
    c = b.get_affine_constant_expr
    zero = F.AffineMap.get(0, 0, [c(0), c(0)], ctx)
    map_c = F.AffineMap.get(2, 0, [d0 * c(TM), d1 * c(TN)], ctx)
    if accumulate:
        b.create_copy_op(C, acc, [by, bx], [], map_c, zero, [TM, TN], [TM, TN])
    elif tweak != "no_init":
        b.create_fill_op(acc, 1.0 if tweak == "fill_one" else 0.0, dtype)

    def loop(_, k):
        # k runs over 0, kstep, 2 kstep, ...: slice k / kstep starts at K offset (k / kstep) * TK
        per_k = TK // kstep if tweak != "k_gap" else 2 * TK // kstep
        map_a = F.AffineMap.get(2, 0, [d0 * c(TM), d1 * c(per_k)], ctx)
        map_b = F.AffineMap.get(2, 0, [d0 * c(per_k), d1 * c(TN)], ctx)
        row_iv = bx if tweak == "a_rows_follow_bx" else by
        b.create_copy_op(A, sA, [row_iv, k], [], map_a, zero, [TM, TK], [TM, TK])
        b.create_copy_op(B, sB, [k, bx], [], map_b, zero, [TK, TN], [TK, TN])
        if tweak == "extra_fill":
            b.create_fill_op(sA, 0.0, dtype)
        if tweak == "gemm_scaled":
            b.create_gemm_op(sA, sB, acc, False, False, False, sS, sS)
        else:
            b.create_gemm_op(sA, sB, acc, False, tweak == "gemm_trans_b", tweak == "gemm_clears")

    b.create_for_op(0, (K // TK) * kstep, kstep, loop)
    if tweak != "no_store":
        out_map = F.AffineMap.get(2, 0, [d1 * c(TM), d0 * c(TN)], ctx) if tweak == "c_swapped" else map_c
        b.create_copy_op(acc, C, [], [by, bx], zero, out_map, [TM, TN], [TM, TN])
    if row_reduce:
        kind, clear = row_reduce
        Rg = entry.get_argument(3)
        rt = b.create_alloc_buffer_op([TM], dtype, F.MemorySpace.LOCAL).get_result(0)
        b.create_reduce_op(acc, rt, kind, 0 if tweak == "reduce_dim0" else 1, clear)
        zero1 = F.AffineMap.get(0, 0, [c(0)], ctx)
        row_map = F.AffineMap.get(1, 0, [d0 * c(TM if tweak != "reduce_rows_off" else TM + 1)], ctx)
        b.create_copy_op(rt, Rg, [], [by], zero1, row_map, [TM], [TM])
    return module


def build_tiled_reduce(R, C, TR, TC, kind="max", dim=1, dtype="fp16", start="fill", loop=True, tweak=None):
    """The tile-by-tile fold of the reference's online-softmax sketch (tmp/ir.mlir:22-36: a
    frisk.parallel over the rows, a frisk.for over tiles of the row, frisk.copy into a fragment,
    frisk.reduce of the fragment) with the ops the builder has: a [R, C] GLOBAL source reduced over
    `dim` into a GLOBAL vector.  `start`: "fill" (the accumulator starts at the kind's identity),
    "load" (it starts from the destination: clear = false for the whole reduce), "reduce_clears"
    (single tile, the reduce op clears)."""
    ctx = F.context()
    F.frisk.load_dialects(ctx)
    b = F.builder(ctx)
    module = b.create_module()
    module.context = ctx
    ty = {"fp16": b.get_f16_ty, "bf16": b.get_bf16_ty, "fp32": b.get_f32_ty}[dtype]()
    mk = lambda shape: b.get_memref_ty(ty, shape, F.AffineMap(), F.MemorySpace.GLOBAL)
    keep = 1 - dim
    shape, T = [R, C], [TR, TC]
    kernel = b.create_kernel_op(module, "fold", b.get_kernel_ty([mk(shape), mk([shape[keep]])]))
    module.push_back(kernel)
    entry = kernel.add_entry_block()
    b.set_insertion_point_to_start(entry)
    X, Y = entry.get_argument(0), entry.get_argument(1)
    grid = shape[keep] // T[keep] - (1 if tweak == "grid_short" else 0)
    par = b.create_parallel_op([grid], 128)
    body = par.add_entry_block()
    b.set_insertion_point_to_start(body)
    blk = body.get_argument(0)
    x = b.create_alloc_buffer_op(T, dtype, F.MemorySpace.LOCAL).get_result(0)
    m = b.create_alloc_buffer_op([T[keep]], dtype, F.MemorySpace.LOCAL).get_result(0)
    d0, d1 = b.get_affine_dim_expr(0), b.get_affine_dim_expr(1)
    c = b.get_affine_constant_expr
    zero2 = F.AffineMap.get(0, 0, [c(0), c(0)], ctx)
    zero1 = F.AffineMap.get(0, 0, [c(0)], ctx)
    place = F.AffineMap.get(1, 0, [d0 * c(T[keep] + (1 if tweak == "result_off" else 0))], ctx)
    identity = {"add": 0.0, "mul": 1.0, "min": float("inf"), "max": float("-inf")}[kind]
    if start == "fill":
        b.create_fill_op(m, 0.5 if tweak == "fill_other" else identity, dtype)
    elif start == "load":
        b.create_copy_op(Y, m, [blk], [], place, zero1, [T[keep]], [T[keep]])
    op_clear = start == "reduce_clears" or tweak == "reduce_clears_in_loop"

    def tile(iv):
        # the source tile: the kept dimension follows the block index, the reduced one the loop
        step = T[dim] * (2 if tweak == "gap" else 1)
        if iv is None:
            exprs = [d0 * c(T[keep]), c(0)] if dim == 1 else [c(0), d0 * c(T[keep])]
            src_map, idx = F.AffineMap.get(1, 0, exprs, ctx), [blk]
        else:
            exprs = [d0 * c(T[0]), d1 * c(step)] if dim == 1 else [d1 * c(step), d0 * c(T[1])]
            src_map, idx = F.AffineMap.get(2, 0, exprs, ctx), [blk, iv]
        b.create_copy_op(X, x, idx, [], src_map, zero2, T, T)
        if tweak == "extra_fill":
            b.create_fill_op(x, 0.0, dtype)
        b.create_reduce_op(x, m, kind, dim, op_clear)

    if loop:
        b.create_for_op(0, shape[dim] // T[dim], 1, lambda _, iv: tile(iv))
    else:
        tile(None)
    if tweak != "no_store":
        b.create_copy_op(m, Y, [], [blk], zero1, place, [T[keep]], [T[keep]])
    return module
