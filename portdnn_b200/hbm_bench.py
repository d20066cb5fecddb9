"""Achieved bandwidth of the HBM-bound operators (depthwise convolution, pooling, pointwise, bias) on
the shapes of the benchmark networks: CUDA events, 20 launches after 3 warm-ups, algorithmic bytes
(every tensor once) / time.

    python -m portdnn_b200.hbm_bench
"""
import sys, os
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import torch
import portdnn_b200 as pd
from portdnn_b200 import workloads
def timeit(fn, reps=20):
    for _ in range(3): fn()
    torch.cuda.synchronize()
    e0,e1=torch.cuda.Event(enable_timing=True),torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps): fn()
    e1.record(); torch.cuda.synchronize()
    return e0.elapsed_time(e1)/reps
res=[]
# depthwise MobileNet-v2 N=128 fp16 forward
tot_b=0; tot_ms=0
for p in workloads.mobilenet_v2_depthwise(128):
    x=torch.randn(p.batch*p.in_rows*p.in_cols*p.channels,device='cuda').half()
    w=torch.randn(9*p.channels,device='cuda').half()
    y=torch.empty(p.batch*p.out_rows*p.out_cols*p.channels,device='cuda').half()
    ms=timeit(lambda: pd.depthwise_conv2d(pd.FORWARD,x,w,p,out=y))
    b=2*(x.numel()+w.numel()+y.numel()); tot_b+=b; tot_ms+=ms
    res.append(("dw_fwd %dx%dx%d s%d"%(p.in_rows,p.in_cols,p.channels,p.stride_rows), ms, b/ms/1e6))
res.append(("dw_fwd mobilenet_v2 total", tot_ms, tot_b/tot_ms/1e6))
# depthwise input-bp and filter-bp on two layers
for (s,c,st) in ((112,96,2),(56,144,1),(14,384,1)):
    p=pd.depthwise_params(128,s,s,c,1,3,st)
    x=torch.randn(p.batch*s*s*c,device='cuda').half(); w=torch.randn(9*c,device='cuda').half()
    dy=torch.randn(p.batch*p.out_rows*p.out_cols*c,device='cuda').half()
    dx=torch.empty_like(x); dw=torch.empty_like(w)
    ms=timeit(lambda: pd.depthwise_conv2d(pd.INPUT_BACKPROP,dy,w,p,out=dx)); res.append(("dw_ibp %dx%d s%d"%(s,c,st), ms, 2*(x.numel()+w.numel()+dy.numel())/ms/1e6))
    ms=timeit(lambda: pd.depthwise_conv2d(pd.FILTER_BACKPROP,x,dy,p,out=dw)); res.append(("dw_fbp %dx%d s%d"%(s,c,st), ms, 2*(x.numel()+w.numel()+dy.numel())/ms/1e6))
# pooling
for name,(n,h,c,win,st,same,dt,op) in {"resnet_stem_maxpool f16":(256,112,64,3,2,True,torch.float16,pd.POOL_MAX),
        "vgg_pool1 f32":(64,224,64,2,2,False,torch.float32,pd.POOL_MAX),"vgg_pool3 f32":(64,56,256,2,2,False,torch.float32,pd.POOL_MAX),
        "resnet_global_avg f16":(256,7,2048,7,1,False,torch.float16,pd.POOL_AVERAGE)}.items():
    p=pd.pool_params(n,h,h,c,win,st,same)
    x=torch.randn(n*h*h*c,device='cuda').to(dt); y=torch.empty(n*p.out_rows*p.out_cols*c,device='cuda',dtype=dt)
    es=x.element_size()
    ms=timeit(lambda: pd.pooling(op,0,x,p,out=y)); res.append(("pool_fwd "+name, ms, es*(x.numel()+y.numel())/ms/1e6))
    dy=torch.randn_like(y); dx=torch.empty_like(x)
    if op==pd.POOL_MAX:
        ms=timeit(lambda: pd.pooling_max_grad(op,x,y,dy,p,out=dx)); res.append(("pool_maxgrad "+name, ms, es*(2*x.numel()+2*y.numel())/ms/1e6))
    else:
        ms=timeit(lambda: pd.pooling(op,1,dy,p,out=dx)); res.append(("pool_avggrad "+name, ms, es*(x.numel()+y.numel())/ms/1e6))
# pointwise / bias
n=256*56*56*256
x=torch.randn(n,device='cuda').half(); y=torch.empty_like(x); b=torch.randn(256,device='cuda').half()
ms=timeit(lambda: pd.pointwise(pd.ACT_RELU,x,out=y)); res.append(("relu_fwd f16 411MB", ms, 4*n/ms/1e6))
ms=timeit(lambda: pd.pointwise_grad(pd.ACT_RELU,x,y,out=y)); res.append(("relu_grad f16", ms, 6*n/ms/1e6))
ms=timeit(lambda: pd.pointwise(pd.ACT_TANH,x,out=y)); res.append(("tanh_fwd f16", ms, 4*n/ms/1e6))
ms=timeit(lambda: pd.bias_add(x,b,256,activation=pd.ACT_RELU,out=y)); res.append(("bias_relu f16", ms, 4*n/ms/1e6))
# binary operators: equal shapes (a residual add), per-channel row (the bias form), per-image per-channel scale
z=torch.randn(n,device='cuda').half(); se=torch.rand(256*256,device='cuda').half()
ms=timeit(lambda: pd.binaryop(pd.BINARY_ADD,x,[256,56,56,256],z,[256,56,56,256],out=y)); res.append(("binary add, equal shapes f16", ms, 6*n/ms/1e6))
ms=timeit(lambda: pd.binaryop(pd.BINARY_MUL,x,[256*56*56,256],b,[1,256],out=y)); res.append(("binary mul, [rows,C] x [1,C] f16", ms, 4*n/ms/1e6))
ms=timeit(lambda: pd.binaryop(pd.BINARY_MUL,x,[256,56*56,256],se,[256,1,256],out=y)); res.append(("binary mul, [N,HW,C] x [N,1,C] f16", ms, 4*n/ms/1e6))
xa=x.abs()
ms=timeit(lambda: pd.pointwise(pd.PW_SQRT,xa,out=y)); res.append(("sqrt_fwd f16", ms, 4*n/ms/1e6))
# batchnorm (ResNet stage-1 activation, fp16) and softmax (ImageNet classifier head)
nb,hb,cb=256,56,256
xb=torch.randn(nb*hb*hb*cb,device='cuda').half(); dyb=torch.randn_like(xb)
beta,gamma,mean=(torch.randn(cb,device='cuda').half() for _ in range(3)); var=(torch.rand(cb,device='cuda')+0.5).half()
yb=torch.empty_like(xb)
for training in (False, True):
    pb=pd.batchnorm_params(nb,hb,hb,cb,training)
    tag="training" if training else "frozen"
    ms=timeit(lambda: pd.batchnorm_forward(xb,beta,gamma,mean,var,pb,out=yb)); res.append(("batchnorm_fwd %s f16 411MB"%tag, ms, (4 if not training else 8)*xb.numel()/ms/1e6))
    ms=timeit(lambda: pd.batchnorm_gradient(xb,dyb,gamma,pb,pop_mean=mean,pop_variance=var,out=yb)); res.append(("batchnorm_grad %s f16"%tag, ms, (10 if training else 8)*xb.numel()/ms/1e6))
xs=torch.randn(4096*1000,device='cuda').half(); ys=torch.empty_like(xs)
ms=timeit(lambda: pd.softmax(xs,4096,1,1,1000,out=ys)); res.append(("softmax_fwd 4096x1000 f16 (8 MB, L2)", ms, 4*xs.numel()/ms/1e6))
xs2=torch.randn(64*56*56*256,device='cuda').half(); ys2=torch.empty_like(xs2)
ms=timeit(lambda: pd.softmax(xs2,64,56,56,256,out=ys2)); res.append(("softmax_fwd 64x56x56x256 f16", ms, 4*xs2.numel()/ms/1e6))
for r in res: print("%-40s %8.4f ms %8.0f GB/s"%r)
