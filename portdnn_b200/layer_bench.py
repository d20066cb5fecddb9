"""Times one forward convolution layer (fused bias + ReLU) a few times with CUDA events; also the
small, self-contained workload used for profiler captures of the implicit-GEMM kernel.

    python -m portdnn_b200.layer_bench N H W C K WINDOW STRIDE [f16|bf16|f32] [reps]
"""
import sys, os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import portdnn_b200 as pd
n,h,w,c,k,win,st = [int(v) for v in sys.argv[1:8]]
dt = {"f16":torch.float16,"bf16":torch.bfloat16,"f32":torch.float32}[sys.argv[8] if len(sys.argv)>8 else "f16"]
reps = int(sys.argv[9]) if len(sys.argv)>9 else 3
p = pd.conv_params(n,h,w,c,k,win,st)
x = torch.randn(n*h*w*c, device='cuda').to(dt)
wt = (torch.randn(win*win*c*k, device='cuda')*(2.0/(win*win*c))**0.5).to(dt)
b = torch.zeros(k, device='cuda').to(dt)
y = torch.empty(n*p.out_rows*p.out_cols*k, device='cuda', dtype=dt)
evs=[]
for i in range(reps):
    e0,e1=torch.cuda.Event(enable_timing=True),torch.cuda.Event(enable_timing=True)
    e0.record(); pd.conv2d(pd.FORWARD, x, wt, p, algorithm=pd.ALGO_TILED, out=y, bias=b, activation=pd.ACT_RELU); e1.record()
    evs.append((e0,e1))
torch.cuda.synchronize()
fl = 2*n*p.out_rows*p.out_cols*win*win*c*k
for e0,e1 in evs:
    ms=e0.elapsed_time(e1); print("ms %.4f  TFLOP/s %.1f" % (ms, fl/ms/1e9))
print("err", pd.device_error_record())
