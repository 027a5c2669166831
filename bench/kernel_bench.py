"""Per-kernel roofline benchmark: GEMM (vs torch.matmul), FlashAttention (vs torch SDPA), norm, cross
entropy and Adam bandwidth.  CUDA-event timing, 3 warm-ups, L2 flushed between iterations.

    python bench/kernel_bench.py            # full sweep
    python bench/kernel_bench.py --small    # one small GEMM + attention call (sized for an ncu capture)
    python bench/kernel_bench.py --attn-llama   # attention at the Llama-7B tensor-parallel shapes vs SDPA
"""
import torch, sys, time
import os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from rumus_b200.ops import native, functional as F
def timeit(fn, n=10, warm=3):
    for _ in range(warm): fn()
    torch.cuda.synchronize()
    flush = torch.empty(256<<20, dtype=torch.uint8, device='cuda')
    ts=[]
    for _ in range(n):
        flush.zero_()
        s=torch.cuda.Event(enable_timing=True); e=torch.cuda.Event(enable_timing=True)
        s.record(); fn(); e.record(); torch.cuda.synchronize(); ts.append(s.elapsed_time(e))
    ts.sort(); return ts[len(ts)//2]
if "--attn-llama" in sys.argv:
    # FlashAttention forward / backward against torch SDPA at B 2, S 4096, D 128 with 16 and 8 local heads
    # (Llama-7B under 2- and 4-way tensor parallelism)
    import torch.nn.functional as TF
    for (B, S, H) in ((2, 4096, 16), (2, 4096, 8)):
        D = 128
        q, k, v = [(torch.randn(B, S, H, D, device='cuda') * 0.5).bfloat16().requires_grad_(True) for _ in range(3)]
        fl = 4 * B * H * S * S * D / 2
        t = timeit(lambda: F.flash_attention(q, k, v, True)); print(f"B{B} S{S} H{H} fwd ours {t:.3f} ms {fl/t/1e9:.0f} TF")
        o = F.flash_attention(q, k, v, True); do = torch.randn_like(o)
        def bw():
            q.grad = k.grad = v.grad = None; o.backward(do, retain_graph=True)
        t = timeit(bw); print(f"   bwd ours {t:.3f} ms {2.5*fl/t/1e9:.0f} TF")
        qt, kt, vt = [x.detach().transpose(1, 2).requires_grad_(True) for x in (q, k, v)]
        t = timeit(lambda: TF.scaled_dot_product_attention(qt, kt, vt, is_causal=True)); print(f"   fwd sdpa {t:.3f} ms {fl/t/1e9:.0f} TF")
        ot = TF.scaled_dot_product_attention(qt, kt, vt, is_causal=True); dot = torch.randn_like(ot)
        def bw2():
            qt.grad = kt.grad = vt.grad = None; ot.backward(dot, retain_graph=True)
        t = timeit(bw2); print(f"   bwd sdpa {t:.3f} ms {2.5*fl/t/1e9:.0f} TF")
    print("status", native.read_status())
    sys.exit(0)
if "--gemm-compare" in sys.argv:
    # one GEMM shape through the one-CTA kernel, the two-CTA kernel and torch.matmul, a few launches
    # each (sized for a counter capture: python bench/kernel_bench.py --gemm-compare M N K)
    i = sys.argv.index("--gemm-compare")
    M, N, K = (int(v) for v in sys.argv[i + 1:i + 4])
    a = torch.randn(M, K, device='cuda').bfloat16(); b = torch.randn(K, N, device='cuda').bfloat16()
    for _ in range(3):
        native.gemm(a, b, path=1, bn=256)
    for mt in (1, 2):
        for _ in range(3):
            native.gemm(a, b, path=3, mt=mt)
    for _ in range(3):
        torch.matmul(a, b)
    torch.cuda.synchronize()
    print("gemm compare done, status", native.read_status())
    sys.exit(0)
if "--small" in sys.argv:
    a = torch.randn(8192, 4096, device='cuda').bfloat16(); b = torch.randn(4096, 8192, device='cuda').bfloat16()
    for _ in range(3):
        native.gemm(a, b, path=1, bn=256)
    B, S, H, D = 2, 2048, 16, 128
    q, k, v = [(torch.randn(B, S, H, D, device='cuda') * 0.5).bfloat16().requires_grad_(True) for _ in range(3)]
    o = F.flash_attention(q, k, v, True)
    o.backward(torch.randn_like(o))
    # LayerNorm forward (with the residual add) and backward (with the residual-stream gradient), 16384 x 2048
    x = torch.randn(16384, 2048, device='cuda').bfloat16(); r = torch.randn_like(x)
    g = torch.ones(2048, device='cuda').bfloat16(); bb = torch.zeros(2048, device='cuda').bfloat16()
    for _ in range(2):
        y, h, stats = native.norm_fwd(x, g, bb, 1e-5, False, residual=r)
        native.norm_bwd(h, y, g, stats, False, dres=r)
    torch.cuda.synchronize()
    print("small case done, status", native.read_status())
    sys.exit(0)
print("== GEMM bf16 (TFLOP/s): mine vs torch.matmul")
for (M,N,K,bt) in [(16384,2048,2048,False),(16384,6144,2048,False),(16384,8192,2048,False),(16384,2048,8192,False),(16384,50304,2048,False),(8192,8192,8192,False),(16384,2048,8192,True)]:
    a=torch.randn(M,K,device='cuda').bfloat16(); 
    bs=torch.randn((N,K) if bt else (K,N),device='cuda').bfloat16(); b=bs.t() if bt else bs
    t=timeit(lambda: native.gemm(a,b)); print(f"M{M} N{N} K{K} bt={bt} default (CTA pairs): {t:.3f} ms {2*M*N*K/t/1e9:.0f} TF", flush=True)
    t=timeit(lambda: native.gemm(a,b,path=1,bn=256)); print(f"   one-CTA 128x256: {t:.3f} ms {2*M*N*K/t/1e9:.0f} TF", flush=True)
    t=timeit(lambda: torch.matmul(a,b)); print(f"   torch: {t:.3f} ms {2*M*N*K/t/1e9:.0f} TF", flush=True)
    st=native.read_status(); assert st==0, st
# wgrad-like: A^T B
M,N,K=2048,8192,16384
x=torch.randn(K,M,device='cuda').bfloat16(); dy=torch.randn(K,N,device='cuda').bfloat16()
t=timeit(lambda: native.gemm(x.t(),dy)); print(f"wgrad M{M} N{N} K{K} default (CTA pairs): {t:.3f} ms {2*M*N*K/t/1e9:.0f} TF")
t=timeit(lambda: torch.matmul(x.t(),dy)); print(f"   torch: {t:.3f} ms {2*M*N*K/t/1e9:.0f} TF")
print("== FlashAttention fwd/bwd B8 H16 S2048 D128 causal")
B,S,H,D=8,2048,16,128
q,k,v=[(torch.randn(B,S,H,D,device='cuda')*0.5).bfloat16().requires_grad_(True) for _ in range(3)]
fl=4*B*H*S*S*D/2
t=timeit(lambda: F.flash_attention(q,k,v,True)); print(f"fwd mine {t:.3f} ms {fl/t/1e9:.0f} TF")
o=F.flash_attention(q,k,v,True); do=torch.randn_like(o)
def bw():
    q.grad=k.grad=v.grad=None
    o.backward(do, retain_graph=True)
t=timeit(bw); print(f"bwd mine {t:.3f} ms {2.5*fl/t/1e9:.0f} TF")
print("status", native.read_status())
import torch.nn.functional as TF
qt,kt,vt=[x.detach().transpose(1,2).requires_grad_(True) for x in (q,k,v)]
t=timeit(lambda: TF.scaled_dot_product_attention(qt,kt,vt,is_causal=True)); print(f"fwd torch sdpa {t:.3f} ms {fl/t/1e9:.0f} TF")
ot=TF.scaled_dot_product_attention(qt,kt,vt,is_causal=True); dot=torch.randn_like(ot)
def bw2():
    qt.grad=kt.grad=vt.grad=None
    ot.backward(dot, retain_graph=True)
t=timeit(bw2); print(f"bwd torch sdpa {t:.3f} ms {2.5*fl/t/1e9:.0f} TF")
print("== norm / CE / adam bandwidth")
x=torch.randn(16384,2048,device='cuda').bfloat16(); g=torch.ones(2048,device='cuda').bfloat16(); bb=torch.zeros(2048,device='cuda').bfloat16()
t=timeit(lambda: native.norm_fwd(x,g,bb,1e-5,False)); print(f"LN fwd {t*1e3:.0f} us {2*x.numel()*2/t/1e6:.0f} GB/s")
y,_,stats=native.norm_fwd(x,g,bb,1e-5,False)
t=timeit(lambda: native.norm_bwd(x,y,g,stats,False)); print(f"LN bwd {t*1e3:.0f} us {3*x.numel()*2/t/1e6:.0f} GB/s")
lg=torch.randn(16384,50304,device='cuda').bfloat16(); tg=torch.randint(0,50304,(16384,),device='cuda')
t=timeit(lambda: native.cross_entropy(lg,tg,1.0,1.0,True,inplace=False)); print(f"CE fwd+bwd {t*1e3:.0f} us {3*lg.numel()*2/t/1e6:.0f} GB/s")
n=300_000_000
p=torch.zeros(n,device='cuda'); m=torch.zeros(n,device='cuda'); vv=torch.zeros(n,device='cuda'); gg=torch.zeros(n,device='cuda').bfloat16(); mm=torch.zeros(n,device='cuda').bfloat16()
t=timeit(lambda: native.adam_flat(gg,p,m,vv,mm,lr=1e-3,beta1=0.9,beta2=0.999,eps=1e-8,weight_decay=0.0,step=1,adamw=False)); print(f"adam flat {t*1e3:.0f} us {n*(2+24+2)/t/1e6:.0f} GB/s")
