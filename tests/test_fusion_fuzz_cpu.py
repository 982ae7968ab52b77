"""Random small graphs over the operators the fusion rewrites look at (Mul, Add, Neg, Slice, Concat,
ReduceMean, 1x1 Conv, Sigmoid, the exported rotary and squeeze-and-excite shapes and near misses of
them) through both planners with the rewrites on: every graph must plan without an error, nothing
may be left dangling, and the rewrites must actually fire somewhere in the corpus."""
import collections
import random

import numpy as np

from fluidml_b200 import models
from fluidml_b200.executor import Executor

FLOAT = 1


def build(seed):
    rnd=random.Random(seed)
    g=models.GraphBuilder(f"f{seed}")
    N,C,H,W=rnd.choice([(1,8,4,4),(2,16,6,6),(1,8,1,1),(2,4,8,8)])
    vals=[g.input("x0",FLOAT,(N,C,H,W)), g.input("x1",FLOAT,(N,C,H,W))]
    gates=[g.input("g0",FLOAT,(N,C,1,1))]
    for step in range(rnd.randint(3,14)):
        op=rnd.choice(["mul","add","neg","slicecat","mean","conv","relu","sig","mulgate","rot"])
        a=rnd.choice(vals); b=rnd.choice(vals)
        sa=g.shapes[a]
        try:
            if op=="mul" and g.shapes[a]==g.shapes[b]: vals.append(g.mul(a,b))
            elif op=="add" and g.shapes[a]==g.shapes[b]: vals.append(g.add(a,b))
            elif op=="neg": vals.append(g.neg(a))
            elif op=="relu": vals.append(g.relu(a))
            elif op=="sig": vals.append(g.sigmoid(a))
            elif op=="slicecat" and sa[3]>=4:
                h=sa[3]//2
                lo=g.slice(a,[0],[h],[3]); hi=g.slice(a,[h],[sa[3]],[3])
                vals.append(g.concat(g.neg(hi) if rnd.random()<0.5 else hi, lo, 3))
            elif op=="mean":
                m=g.reduce_mean(a,[2,3]); gates.append(m)
                cr=max(1,sa[1]//4)
                w1=g.const(f"w1_{step}",np.ones((cr,sa[1],1,1),np.float32)); w2=g.const(f"w2_{step}",np.ones((sa[1],cr,1,1),np.float32))
                h1=g.conv(m,w1,None,pads=[0]*4,strides=[1,1],dilations=[1,1],group=1)
                if rnd.random()<0.5: h1=g.mul(h1,g.sigmoid(h1))
                h2=g.conv(h1,w2,None,pads=[0]*4,strides=[1,1],dilations=[1,1],group=1)
                if rnd.random()<0.7: h2=g.sigmoid(h2)
                vals.append(g.mul(a,h2))
            elif op=="conv":
                oc=rnd.choice([4,8,16])
                w=g.const(f"w_{step}",np.ones((oc,sa[1],1,1),np.float32))
                y=g.conv(a,w,None,pads=[0]*4,strides=[1,1],dilations=[1,1],group=1)
                if g.shapes[y]==g.shapes[vals[0]]: vals.append(y)
            elif op=="mulgate":
                gt=rnd.choice(gates)
                if g.shapes[gt][:2]==sa[:2]: vals.append(g.mul(a,gt))
            elif op=="rot" and sa[3]>=8:
                rot=sa[3]//2; half=rot//2
                cs=g.const(f"c_{step}",np.ones((sa[2],rot),np.float32)); sn=g.const(f"s_{step}",np.ones((sa[2],rot),np.float32))
                xr=g.slice(a,[0],[rot],[3]); xp=g.slice(a,[rot],[sa[3]],[3])
                hi=g.slice(xr,[half],[rot],[3]); lo=g.slice(xr,[0],[half],[3])
                y=g.add(g.mul(xr,cs),g.mul(g.concat(g.neg(hi),lo,3),sn))
                vals.append(g.concat(y,xp,3))
        except Exception as e:
            pass
        vals=[v for v in vals if v is not None]
    # sum everything of the base shape into the output so nothing is dead
    base=[v for v in vals if g.shapes[v]==g.shapes[vals[0]]]
    acc=base[0]
    for v in base[1:]: acc=g.add(acc,v)
    g.relu(acc,out="y"); g.output("y")
    return g.finish()


def test_random_graphs_plan_with_every_rewrite_on():
    seen = collections.Counter()
    built = 0
    for seed in range(80):
        try:
            m = build(seed)
        except Exception:
            continue  # the generator drew an ill-formed graph
        built += 1
        for factory in (Executor.make_plain_greedy, Executor.make_dp_greedy):
            st = factory("fuzz").plan(m.to_bytes())
            outs = [n["output"] for n in st["sequence"]]
            assert len(outs) == len(set(outs)) and "y" in outs, seed
            for n in st["sequence"]:
                seen[n["kind"]] += 1
    assert built >= 60
    assert seen["SqueezeExciteGate"] > 0 and seen["Rotary"] > 0 and seen["FusedMulAdd"] > 0
