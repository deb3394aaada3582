//! Binding tests, to run on a machine with a Rust toolchain and a B200: the calls a `compute()` makes, through
//! the safe wrappers, checked against host arithmetic.  The same calls with the same conventions are covered
//! through ctypes by tests/test_gpu_abi_ops.py in this repository.
use sage_cuda_backend::backend::cuda::{CudaBackend, CudaMemory};
use sage_cuda_backend::backend::{Backend, DataType, ReduceKind, TensorView};

fn bytes(v: &[f32]) -> &[u8] {
    unsafe { std::slice::from_raw_parts(v.as_ptr() as *const u8, v.len() * 4) }
}
fn read_f32(b: &mut CudaBackend, m: &CudaMemory, n: usize) -> Vec<f32> {
    let mut out = vec![0f32; n];
    let raw = unsafe { std::slice::from_raw_parts_mut(out.as_mut_ptr() as *mut u8, n * 4) };
    b.read(m, raw).unwrap();
    out
}
fn view<'a>(mem: &'a CudaMemory, extents: &'a [usize], strides: &'a [usize], offset: usize) -> TensorView<'a, CudaMemory> {
    TensorView { mem, dtype: DataType::Float, extents, strides, offset }
}

#[test]
fn map_reduce_gemm_round_trip() {
    if CudaBackend::device_list().is_empty() {
        eprintln!("no CUDA device: skipped");
        return;
    }
    let mut b = CudaBackend::with_device(0).unwrap();
    let (r, c) = (64usize, 96usize);
    let x: Vec<f32> = (0..r * c).map(|i| ((i * 37 % 101) as f32) / 50.0 - 1.0).collect();
    let bias: Vec<f32> = (0..c).map(|i| i as f32 * 0.01).collect();
    let (mx, mb, my) = (b.alloc(DataType::Float, r * c).unwrap(), b.alloc(DataType::Float, c).unwrap(), b.alloc(DataType::Float, r * c).unwrap());
    b.write(&mx, bytes(&x)).unwrap();
    b.write(&mb, bytes(&bias)).unwrap();
    // VariadicMapOperator: (x0 * 2 + x1) with x1 broadcast along the rows (stride 0)
    let (e, s, sb) = ([r, c], [c, 1], [0usize, 1]);
    b.map("((x0 * 2.0f) + x1)", &[view(&mx, &e, &s, 0), view(&mb, &e, &sb, 0)], &view(&my, &e, &s, 0)).unwrap();
    let y = read_f32(&mut b, &my, r * c);
    for i in 0..r * c {
        assert_eq!(y[i], x[i] * 2.0 + bias[i % c]);
    }
    // ReduceOperator over axis 1 (the accumulator starts at 0 like the reference's)
    let ms = b.alloc(DataType::Float, r).unwrap();
    b.reduce(ReduceKind::Sum, &view(&my, &e, &s, 0), &[1], &view(&ms, &[r], &[1], 0)).unwrap();
    let sums = read_f32(&mut b, &ms, r);
    for i in 0..r {
        let want: f32 = y[i * c..(i + 1) * c].iter().sum();
        assert!((sums[i] - want).abs() <= 1e-4 * want.abs().max(1.0));
    }
    // Gemm::compute_direct: [r, c] x [c, r] on the tensor cores (3xTF32: fp32 accuracy)
    let mc = b.alloc(DataType::Float, r * r).unwrap();
    let (ea, sa, et, stt, ec, sc) = ([r, c], [c, 1], [c, r], [r, 1], [r, r], [r, 1]);
    let xt: Vec<f32> = (0..c * r).map(|i| x[(i % r) * c + i / r]).collect();
    let mt = b.alloc(DataType::Float, c * r).unwrap();
    b.write(&mt, bytes(&xt)).unwrap();
    b.gemm_batched(false, false, r, r, c, 1, &view(&mx, &ea, &sa, 0), c, 0, &view(&mt, &et, &stt, 0), r, 0, &view(&mc, &ec, &sc, 0), r, 0).unwrap();
    let g = read_f32(&mut b, &mc, r * r);
    for i in 0..r {
        for j in 0..r {
            let want: f64 = (0..c).map(|p| x[i * c + p] as f64 * x[j * c + p] as f64).sum();
            assert!((g[i * r + j] as f64 - want).abs() <= 1e-4 * want.abs().max(1.0));
        }
    }
    assert_eq!(b.status_word().unwrap(), 0);
    // dropping the handles returns the blocks; the pool shows nothing in use
    drop((mx, mb, my, ms, mc, mt));
    assert_eq!(b.mem_stats().mem_used, 0);
}
