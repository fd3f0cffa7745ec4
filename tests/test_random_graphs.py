"""Random autograd graphs (add, mul incl. squares, matmul, reshape, Conv2D, sum; a loss that adds several sums)
built on the device classes and on the oracle: the loss, every node's values and every gradient must agree,
with the loss-graph fusion on and off (crates/katsu-core/src/tensor.rs:226-447 is what both restate).  Seeds are
fixed: 3 x 40 programs."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RNG = None


def rel(a, b):
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    d = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / d) if d > 0 else float(np.linalg.norm(a - b))


def build(lib, program, leaves_data):
    """program: list of (op, args...) referring to earlier values by index; returns all values + layers"""
    vals = [lib.Tensor(d, s) for d, s in leaves_data]
    for step in program:
        op = step[0]
        if op == 'add':
            vals.append(vals[step[1]].add(vals[step[2]]))
        elif op == 'mul':
            vals.append(vals[step[1]].mul(vals[step[2]]))
        elif op == 'matmul':
            vals.append(vals[step[1]].matmul(vals[step[2]]))
        elif op == 'reshape':
            vals.append(vals[step[1]].reshape(step[2]))
        elif op == 'sum':
            vals.append(vals[step[1]].sum())
        elif op == 'conv':
            layer = lib.Conv2D.from_weights(vals[step[2]], step[3], step[4])
            vals.append(layer.forward(vals[step[1]]))
    return vals


def random_program():
    leaves, shapes, program = [], [], []
    def leaf(shape):
        n = int(np.prod(shape))
        leaves.append((RNG.standard_normal(n).astype(np.float32) * np.float32(0.5), list(shape))); shapes.append(list(shape))
        return len(shapes) - 1
    m, k, n = (int(RNG.choice([1, 2, 3, 5, 8, 16])) for _ in range(3))
    a, b, c2 = leaf([m, k]), leaf([k, n]), leaf([m, n])
    # a conv branch
    cin = int(RNG.choice([1, 3, 16])); cout = int(RNG.choice([2, 8, 16])); hh = int(RNG.integers(4, 9)); ww = int(RNG.choice([4, 8]))
    x, w = leaf([int(RNG.integers(1, 3)), cin, hh, ww]), leaf([cout, cin, 3, 3])
    def emit(step, shape):
        program.append(step); shapes.append(list(shape)); return len(shapes) - 1
    scalars = []
    for _ in range(int(RNG.integers(4, 12))):
        choice = RNG.integers(0, 6)
        idxs = list(range(len(shapes)))
        if choice == 0:   # add same shape
            i = int(RNG.choice(idxs)); same = [j for j in idxs if shapes[j] == shapes[i]]
            emit(('add', i, int(RNG.choice(same))), shapes[i])
        elif choice == 1:  # mul same shape (often a square)
            i = int(RNG.choice(idxs)); same = [j for j in idxs if shapes[j] == shapes[i]]
            j = i if RNG.random() < 0.5 else int(RNG.choice(same))
            emit(('mul', i, j), shapes[i])
        elif choice == 2:  # matmul
            r2 = [j for j in idxs if len(shapes[j]) == 2]
            i = int(RNG.choice(r2)); right = [j for j in r2 if shapes[j][0] == shapes[i][1]]
            if right:
                j = int(RNG.choice(right)); emit(('matmul', i, j), [shapes[i][0], shapes[j][1]])
        elif choice == 3:  # reshape to rank 2 or flat
            i = int(RNG.choice(idxs)); numel = int(np.prod(shapes[i])) if shapes[i] else 1
            if numel > 1:
                divs = [d for d in range(1, numel + 1) if numel % d == 0]
                d = int(RNG.choice(divs)); emit(('reshape', i, [d, numel // d]), [d, numel // d])
        elif choice == 4:  # conv with the leaf weights (or a derived tensor of the same shape as w)
            r4 = [j for j in idxs if len(shapes[j]) == 4 and shapes[j][1] == cin and shapes[j][2] >= 2 and shapes[j][3] >= 2 and j != w]
            ws = [j for j in idxs if shapes[j] == shapes[w]]
            if r4:
                i = int(RNG.choice(r4)); wj = int(RNG.choice(ws)); stride = int(RNG.choice([1, 1, 2])); pad = 1
                oh = (shapes[i][2] + 2 - 3) // stride + 1; ow = (shapes[i][3] + 2 - 3) // stride + 1
                emit(('conv', i, wj, stride, pad), [shapes[i][0], cout, oh, ow])
        else:  # sum
            i = int(RNG.choice([j for j in idxs if shapes[j] != []] or idxs))
            scalars.append(emit(('sum', i), []))
    # loss: sum of (possibly squared) sums of a few values
    picks = RNG.choice(len(shapes), size=min(4, len(shapes)), replace=False)
    terms = list(scalars)
    for i in picks:
        i = int(i)
        if shapes[i] == []: terms.append(i); continue
        if RNG.random() < 0.6:
            q = emit(('mul', i, i), shapes[i]); terms.append(emit(('sum', q), []))
        else:
            terms.append(emit(('sum', i), []))
    acc = terms[0]
    for t in terms[1:]:
        acc = emit(('add', acc, t), [])
    return leaves, program, len(leaves)



@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_graphs_match_the_oracle(oracle, seed):
    global RNG
    import katsu_b200 as K

    RNG = np.random.default_rng(seed)
    try:
        for program_index in range(40):
            leaves, program, _ = random_program()
            ref = build(oracle, program, leaves)
            ref[-1].backward()
            scale = max(float(np.abs(r.data()).max()) for r in ref if r.numel() == 1)
            for fusion in (True, False):
                K.set_loss_fusion(fusion)
                dev = build(K, program, leaves)
                dev[-1].backward()
                where = (seed, program_index, fusion, program)
                # the loss may cancel: its error is measured against the largest scalar of the graph
                assert abs(float(dev[-1].data()[0]) - float(ref[-1].data()[0])) <= 2e-5 * max(scale, 1e-30), where
                for i in range(len(ref)):
                    expected, got = ref[i].grad(), dev[i].grad()
                    assert (expected is None) == (got is None), (where, "gradient presence of value", i)
                    if expected is not None:
                        assert rel(got, expected) <= 2e-5, (where, "gradient of value", i)
                    if ref[i].numel() > 1:
                        assert rel(dev[i].data(), ref[i].data()) <= 2e-5, (where, "values of", i)
    finally:
        K.set_loss_fusion(True)
