"""The reference's Linear and matmul known answers (tests/golden/reference_kat.json) expanded into concrete cases,
shared by the oracle's CPU test and the GPU parity test."""
import numpy as np

CODE = {"f32": 0, "f16": 1, "bf16": 2, "i8": 3, "i4": 4, "f8": 5}


def linear_cases(kat):
    """(id, kwargs of oracle.linear_module, expected) for every Linear known answer of the reference."""
    lm = kat["linear_module"]
    f = lm["float"]
    x = np.full(f["input_shape"], f["input_value"], dtype=np.float32)
    w, b = np.array(f["weight"], dtype=np.float32), np.array(f["bias"], dtype=np.float32)
    yield "float", dict(x=x, weight=w, bias=b, code=CODE[f["dtype"]]), np.array(f["expect"], dtype=np.float32)
    q = lm["quant"]
    for qd in q["quant_dtypes"]:
        for dim in q["weight_quant_dims"]:
            for use_in in q["use_input_scale"]:
                n = 1 if dim is None else (q["out_features"] if dim == 0 else q["in_features"])
                ws = np.full((n,) if dim is not None else (), q["scale_value"], dtype=np.float32)
                kw = dict(x=x, weight=w, bias=b, code=CODE[q["dtype"]], quant_code=CODE[qd], weight_quant_dim=dim, weight_scale=ws,
                          input_scale=(q["scale_value"] if use_in else None))
                rejected = use_in == q["rejected"]["use_input_scale"] and dim == q["rejected"]["weight_quant_dim"]
                yield f"{qd}-dim{dim}-in{int(use_in)}", kw, (None if rejected else np.array(q["expect"], dtype=np.float32))
    i4 = lm["int4_weight_only"]
    x4 = np.full(i4["input_shape"], i4["input_value"], dtype=np.float32)
    w4 = np.full((i4["out_features"], i4["in_features"]), i4["weight_value"], dtype=np.float32)
    b4 = np.full((i4["out_features"],), i4["bias_value"], dtype=np.float32)
    for case in i4["cases"]:
        ws = np.full(case["scale_shape"], i4["scale_value"], dtype=np.float32)
        kw = dict(x=x4, weight=w4, bias=b4, code=CODE[i4["dtype"]], quant_code=CODE["i4"], weight_quant_dim=case["weight_quant_dim"], weight_scale=ws)
        yield "int4-" + case["id"], kw, np.full((i4["input_shape"][0], i4["out_features"]), i4["expect_value"], dtype=np.float32)


def iota(shape, dim):
    dim = dim % len(shape)
    idx = np.arange(shape[dim], dtype=np.float32).reshape([-1 if i == dim else 1 for i in range(len(shape))])
    return np.ascontiguousarray(np.broadcast_to(idx, shape))


