"""Per-kernel micro-benchmark of the 'cuda' backend: times one op through the public
op front end with CUDA events on the backend's stream.

    python kernel_bench.py <case> [iterations]

cases: mm2a (fused matMul 4096x1024x4096 + bias + relu6), ffn (8192x768x3072), ffng (ffn with
the erf GELU as epilogue),
mm_<m>_<k>_<n> (fused matMul + bias), qkv_<m>_<k>_<n> (three of them on one activation: one
grouped launch), mean_<batch>_<hw>_<c> (global average pooling), maxpool_<batch>_<hw>_<c> (3x3 stride-2 max pooling), attn_<batch>_<heads>[_sep] (one attention layer, heads of 128 x 64: one launch, or
the three separate ones),
pw_<hw>_<cin>_<cout>_<batch> (1x1 conv), c3_<hw>_<cin>_<cout>_<batch>_<stride> (3x3
conv), stem_<hw>_<k>_<cout>_<batch>_<stride> (3-channel input), dw_<hw>_<c>_<batch>_<stride>
(3x3 depthwise), res_<hw>_<cin>_<cout>_<batch> (1x1 conv + bias, Add of a shortcut, Relu:
one launch through the deferred-launch path), gelu_<rows>_<cols> (x * 0.5 * (1 + erf(x /
sqrt 2)): five elementwise kernels, one catalogued chain launch), ln_<rows>_<cols> (LayerNorm
tail ((x - mean) * rstd) * gamma + beta: four kernels, one chain launch), lnf_<rows>_<cols>
(residual Add + the whole layer normalisation: ten kernels of the reference, one launch),
sm_<rows>_<cols> (softmax of scaled, masked attention scores, rows a multiple of 1536),
dwp_<hw>_<c>_<n>_<batch>_<stride>[_res] (3x3 depthwise + relu6 and the 1x1 projection behind it,
optionally + shortcut: one launch).  Prints ms, TFLOP/s
and algorithmic GB/s (each tensor moved once).
Times are device times of graph replays (n calls per graph, best of three replays).
"""
import sys

import numpy as np

import tfjs_b200
from tfjs_b200 import ops

eng=tfjs_b200.ENGINE; eng.set_backend('cuda'); be=eng.backend
case=sys.argv[1]; iters=int(sys.argv[2]) if len(sys.argv)>2 else 3
r=np.random.default_rng(0)
def timeit(f, n):
    """ms per call: n calls captured into one CUDA graph and the graph replayed, so the
    figure is device time even for kernels shorter than a host-side call (eager launches
    are timed instead when the capture is refused)."""
    for _ in range(2):
        y=f(); be.device_id(y.dataId); nbytes=be.data[y.dataId].nbytes; y.dispose()
    be.sync()
    be.high_water_reset(); y=f(); be.device_id(y.dataId); y.dispose(); be.sync()
    peak=be.memory()['poolHighWater']
    try:
        be.capture_begin(int(peak*1.5)+(16<<20))
        for _ in range(n):
            y=f(); be.device_id(y.dataId); y.dispose()
        graph=be.capture_end(False)
    except Exception:
        try: be.capture_end(True)
        except Exception: pass
        def eager():
            for _ in range(n):
                y=f(); be.device_id(y.dataId); y.dispose()
        return be.time(eager)['kernelMs']/n
    be.graph_launch(graph); be.sync()
    best=min(be.time(lambda: be.graph_launch(graph))['kernelMs'] for _ in range(3))
    be.graph_destroy(graph)
    return best/n
if case=='mm2a':
    a=ops.tensor(r.standard_normal((4096,1024)).astype(np.float32)/32); b=ops.tensor(r.standard_normal((1024,4096)).astype(np.float32)/32)
    bias=ops.tensor(r.standard_normal(4096).astype(np.float32))
    f=lambda: ops.fused_mat_mul(a,b,False,False,bias,'relu6'); fl=2*4096*4096*1024; by=4*(4096*1024*2+4096*4096)
elif case=='ffn':
    a=ops.tensor(r.standard_normal((8192,768)).astype(np.float32)/32); b=ops.tensor(r.standard_normal((768,3072)).astype(np.float32)/32)
    bias=ops.tensor(r.standard_normal(3072).astype(np.float32))
    f=lambda: ops.fused_mat_mul(a,b,False,False,bias,'linear'); fl=2*8192*3072*768; by=4*(8192*768+768*3072+8192*3072)
elif case=='ffng':   # the same product with the erf GELU as its epilogue
    a=ops.tensor(r.standard_normal((8192,768)).astype(np.float32)/32); b=ops.tensor(r.standard_normal((768,3072)).astype(np.float32)/32)
    bias=ops.tensor(r.standard_normal(3072).astype(np.float32))
    f=lambda: ops.fused_mat_mul(a,b,False,False,bias,'gelu_erf',None,0.2,[float(np.float32(1/np.sqrt(2))),0.5,1.0,0.0]); fl=2*8192*3072*768; by=4*(8192*768+768*3072+8192*3072)
elif case.startswith('maxpool_'):   # maxpool_<batch>_<hw>_<c>: 3x3 stride-2 'same' max pooling
    _,bt,hw,c=case.split('_'); bt,hw,c=int(bt),int(hw),int(c)
    x=ops.tensor(r.standard_normal((bt,hw,hw,c)).astype(np.float32))
    f=lambda: ops.max_pool(x,3,2,'same'); fl=0; by=4*(bt*hw*hw*c+bt*((hw+1)//2)**2*c)
elif case.startswith('mean_'):   # mean_<batch>_<hw>_<c>: Mean over the two spatial axes of an NHWC map (global pooling)
    _,bt,hw,c=case.split('_'); bt,hw,c=int(bt),int(hw),int(c)
    x=ops.tensor(r.standard_normal((bt,hw,hw,c)).astype(np.float32))
    f=lambda: ops.mean(x,[1,2]); fl=0; by=4*(bt*hw*hw*c+bt*c)
elif case.startswith('attn_'):   # attn_<batch>_<heads>[_sep]: softmax(q k^T / 8 + mask) v, heads of 128 x 64
    parts=case.split('_'); B,H=int(parts[1]),int(parts[2]); sep=len(parts)>3
    q,k,v=[ops.tensor(r.standard_normal((B,H,128,64)).astype(np.float32)) for _ in range(3)]
    mask=ops.tensor(np.zeros((B,1,1,128),np.float32))
    def f():
        if not sep: return ops.fused_attention(q,k,v,0.125,mask)
        s=ops.mat_mul(q,k,False,True); p=ops.softmax_scaled_masked(s,0.125,mask); o=ops.mat_mul_heads(p,v,'merge',[B,128,H,64])
        be.device_id(o.dataId); s.dispose(); p.dispose(); return o
    fl=4*B*H*128*128*64; by=4*4*B*H*128*64
elif case.startswith('qkv_'):   # qkv_<m>_<k>_<n>: three fused matMuls + bias on one activation (one grouped launch)
    _,m,k,n=case.split('_'); m,k,n=int(m),int(k),int(n)
    a0=ops.tensor(r.standard_normal((m,k)).astype(np.float32)/32); zero=ops.tensor(np.float32(0)); a=ops.add(a0,zero); be.device_id(a.dataId)
    ws=[ops.tensor(r.standard_normal((k,n)).astype(np.float32)/32) for _ in range(3)]
    bs=[ops.tensor(r.standard_normal(n).astype(np.float32)) for _ in range(3)]
    def f():
        ys=[ops.fused_mat_mul(a,w,False,False,b,'linear') for w,b in zip(ws,bs)]
        for y in ys: be.device_id(y.dataId)
        for y in ys[1:]: y.dispose()
        return ys[0]
    fl=3*2*m*n*k; by=4*(m*k+3*k*n+3*m*n)
elif case.startswith('mm_'):   # mm_<m>_<k>_<n>: fused matMul + bias
    _,m,k,n=case.split('_'); m,k,n=int(m),int(k),int(n)
    a=ops.tensor(r.standard_normal((m,k)).astype(np.float32)/32); b=ops.tensor(r.standard_normal((k,n)).astype(np.float32)/32)
    bias=ops.tensor(r.standard_normal(n).astype(np.float32))
    f=lambda: ops.fused_mat_mul(a,b,False,False,bias,'linear'); fl=2*m*n*k; by=4*(m*k+k*n+m*n)
elif case.startswith('gelu'):   # gelu_<rows>_<cols>
    _,rows,cols=case.split('_'); rows,cols=int(rows),int(cols)
    x=ops.tensor(r.standard_normal((rows,cols)).astype(np.float32))
    c=ops.tensor(np.float32(1/np.sqrt(2))); one=ops.tensor(np.float32(1)); half=ops.tensor(np.float32(0.5))
    def f():
        a=ops.mul(x,c); b=ops.erf(a); i=ops.add(b,one); d=ops.mul(x,half); y=ops.mul(d,i)
        be.device_id(y.dataId)
        for t in (a,b,i,d): t.dispose()
        return y
    fl=0; by=8*rows*cols
elif case.startswith('sm_'):   # sm_<rows>_<cols>: softmax(x * 0.125 + mask) with a [rows/1536, 1, 1, cols] mask
    _,rows,cols=case.split('_'); rows,cols=int(rows),int(cols)
    x=ops.tensor(r.standard_normal((rows//1536,12,128,cols)).astype(np.float32)); mask=ops.tensor(np.zeros((rows//1536,1,1,cols),np.float32))
    f=lambda: ops.softmax_scaled_masked(x,0.125,mask); fl=0; by=8*rows*cols
elif case.startswith('lnf'):   # lnf_<rows>_<cols>: residual Add + layer normalisation, one kernel
    _,rows,cols=case.split('_'); rows,cols=int(rows),int(cols)
    x=ops.tensor(r.standard_normal((rows,cols)).astype(np.float32)); res=ops.tensor(r.standard_normal((rows,cols)).astype(np.float32))
    gamma=ops.tensor(r.standard_normal(cols).astype(np.float32)); beta=ops.tensor(r.standard_normal(cols).astype(np.float32))
    f=lambda: ops.fused_layer_norm(x,gamma,beta,1e-12,residual=res); fl=0; by=12*rows*cols
elif case.startswith('ln'):   # ln_<rows>_<cols>
    _,rows,cols=case.split('_'); rows,cols=int(rows),int(cols)
    x=ops.tensor(r.standard_normal((rows,cols)).astype(np.float32)); mean=ops.tensor(r.standard_normal((rows,1)).astype(np.float32))
    rstd=ops.tensor((r.random((rows,1))+0.5).astype(np.float32)); gamma=ops.tensor(r.standard_normal(cols).astype(np.float32)); beta=ops.tensor(r.standard_normal(cols).astype(np.float32))
    def f():
        a=ops.sub(x,mean); b=ops.mul(a,rstd); c2=ops.mul(b,gamma); y=ops.add(c2,beta)
        be.device_id(y.dataId)
        for t in (a,b,c2): t.dispose()
        return y
    fl=0; by=8*rows*cols
elif case.startswith('res'):   # residual block exit: res_<hw>_<cin>_<cout>_<batch>
    _,hw,ci,co,bt=case.split('_'); hw,ci,co,bt=int(hw),int(ci),int(co),int(bt)
    x=ops.tensor(r.standard_normal((bt,hw,hw,ci)).astype(np.float32)); w=ops.tensor(r.standard_normal((1,1,ci,co)).astype(np.float32)/8)
    bias=ops.tensor(r.standard_normal(co).astype(np.float32)); sc=ops.tensor(r.standard_normal((bt,hw,hw,co)).astype(np.float32))
    def f():
        y=ops.fused_conv2d(x,w,1,'same','NHWC',[1,1],None,bias,'linear'); s=ops.add(y,sc); o=ops.relu(s)
        y.dispose(); s.dispose(); return o
    fl=2*bt*hw*hw*ci*co; by=4*(bt*hw*hw*(ci+2*co)+ci*co)
elif case.startswith('pw'):   # pointwise conv: pw_<hw>_<cin>_<cout>_<batch>
    _,hw,ci,co,bt=case.split('_'); hw,ci,co,bt=int(hw),int(ci),int(co),int(bt)
    x=ops.tensor(r.standard_normal((bt,hw,hw,ci)).astype(np.float32)); w=ops.tensor(r.standard_normal((1,1,ci,co)).astype(np.float32)/8)
    bias=ops.tensor(r.standard_normal(co).astype(np.float32))
    f=lambda: ops.fused_conv2d(x,w,1,'same','NHWC',[1,1],None,bias,'relu6'); fl=2*bt*hw*hw*ci*co; by=4*(bt*hw*hw*(ci+co)+ci*co)
elif case.startswith('c3'):   # 3x3 conv: c3_<hw>_<cin>_<cout>_<batch>_<stride>
    _,hw,ci,co,bt,st=case.split('_'); hw,ci,co,bt,st=int(hw),int(ci),int(co),int(bt),int(st)
    x=ops.tensor(r.standard_normal((bt,hw,hw,ci)).astype(np.float32)); w=ops.tensor(r.standard_normal((3,3,ci,co)).astype(np.float32)/24)
    bias=ops.tensor(r.standard_normal(co).astype(np.float32))
    f=lambda: ops.fused_conv2d(x,w,st,'same','NHWC',[1,1],None,bias,'relu'); ho=(hw+st-1)//st; fl=2*bt*ho*ho*9*ci*co; by=4*(bt*hw*hw*ci+bt*ho*ho*co+9*ci*co)
elif case.startswith('stem'):   # stem_<hw>_<k>_<cout>_<batch>_<stride>
    _,hw,k,co,bt,st=case.split('_'); hw,k,co,bt,st=int(hw),int(k),int(co),int(bt),int(st)
    x=ops.tensor(r.standard_normal((bt,hw,hw,3)).astype(np.float32)); w=ops.tensor(r.standard_normal((k,k,3,co)).astype(np.float32)/8)
    bias=ops.tensor(r.standard_normal(co).astype(np.float32))
    f=lambda: ops.fused_conv2d(x,w,st,'same','NHWC',[1,1],None,bias,'relu6'); ho=(hw+st-1)//st; fl=2*bt*ho*ho*k*k*3*co; by=4*(bt*hw*hw*3+bt*ho*ho*co)
elif case.startswith('dw_'):   # depthwise: dw_<hw>_<c>_<batch>_<stride>
    _,hw,c,bt,st=case.split('_'); hw,c,bt,st=int(hw),int(c),int(bt),int(st)
    x=ops.tensor(r.standard_normal((bt,hw,hw,c)).astype(np.float32)); w=ops.tensor(r.standard_normal((3,3,c,1)).astype(np.float32)/3)
    bias=ops.tensor(r.standard_normal(c).astype(np.float32))
    f=lambda: ops.fused_depthwise_conv2d(x,w,st,'same','NHWC',[1,1],None,bias,'relu6'); ho=(hw+st-1)//st; fl=2*bt*ho*ho*9*c; by=4*(bt*hw*hw*c+bt*ho*ho*c)
elif case.startswith('dwp'):   # dwp_<hw>_<c>_<n>_<batch>_<stride>[_res]: 3x3 depthwise + relu6, then 1x1 projection (+ shortcut)
    parts=case.split('_'); hw,c,n,bt,st=[int(v) for v in parts[1:6]]; res=len(parts)>6
    x=ops.tensor(r.standard_normal((bt,hw,hw,c)).astype(np.float32)); wd=ops.tensor(r.standard_normal((3,3,c,1)).astype(np.float32)/3)
    bd=ops.tensor(r.standard_normal(c).astype(np.float32)); wp=ops.tensor(r.standard_normal((1,1,c,n)).astype(np.float32)/8)
    bp=ops.tensor(r.standard_normal(n).astype(np.float32)); ho=(hw+st-1)//st
    sc=ops.tensor(r.standard_normal((bt,ho,ho,n)).astype(np.float32)) if res else None
    def f():
        h=ops.fused_depthwise_conv2d(x,wd,st,'same','NHWC',[1,1],None,bd,'relu6')
        y=ops.fused_conv2d(h,wp,1,'same','NHWC',[1,1],None,bp,'linear'); h.dispose()
        if sc is not None:
            s2=ops.add(sc,y); y.dispose(); y=s2
        return y
    fl=2*bt*ho*ho*c*(9+n); by=4*(bt*hw*hw*c+bt*ho*ho*n*(2 if res else 1))
ms=timeit(f,iters)
print('%s: %.4f ms  %.1f TFLOP/s  %.1f GB/s (algorithmic)'%(case,ms,fl/ms/1e9,by/ms/1e6))
