//! The glue a `b200` cargo feature of autograph would add next to its krnl code: a device
//! handle, an owning buffer, and the bodies that replace the krnl dispatch blocks.
//! NOT COMPILED where this repository is developed (no Rust toolchain on those machines); the C
//! entry points it calls are exercised by tests/ (Python, and plain C in tests/c_driver/).
//!
//! Each function names the reference site it stands in for (path:line inside autograph).

use anyhow::{bail, Result};
use autograph_b200_sys as sys;
use std::os::raw::{c_int, c_void};
use std::sync::Arc;

/// ≙ krnl's `Device` for this backend (Device::builder().index(i).build(),
/// tests/integration_tests.rs:27-30).  Calls on one device run in submission order.
#[derive(Clone)]
pub struct Device(Arc<DeviceInner>);
struct DeviceInner(*mut sys::ag_device);
unsafe impl Send for DeviceInner {}
unsafe impl Sync for DeviceInner {}
impl Drop for DeviceInner {
    fn drop(&mut self) {
        unsafe { sys::ag_device_destroy(self.0) };
    }
}
impl Device {
    pub fn new(index: usize) -> Result<Self> {
        let mut raw = std::ptr::null_mut();
        sys::check(unsafe { sys::ag_device_create(index as c_int, &mut raw) })?;
        Ok(Self(Arc::new(DeviceInner(raw))))
    }
    pub fn raw(&self) -> *mut sys::ag_device {
        self.0 .0
    }
    /// ≙ device.wait() (src/tensor/linalg.rs:549)
    pub fn wait(&self) -> Result<()> {
        sys::check(unsafe { sys::ag_device_wait(self.raw()) })
    }
}

/// ≙ krnl's `Buffer<T>` on the device: owns `len` elements of device memory
/// (Tensor::into_device / into_array, src/tensor.rs:1819-1833, 1923-1945).
pub struct Buffer<T> {
    device: Device,
    ptr: *mut c_void,
    len: usize,
    _marker: std::marker::PhantomData<T>,
}
impl<T: Copy> Buffer<T> {
    pub fn zeros(device: Device, len: usize) -> Result<Self> {
        let mut ptr = std::ptr::null_mut();
        let bytes = len * std::mem::size_of::<T>();
        sys::check(unsafe { sys::ag_alloc(device.raw(), bytes, &mut ptr) })?;
        sys::check(unsafe { sys::ag_fill_zero(device.raw(), ptr, bytes) })?;
        Ok(Self { device, ptr, len, _marker: Default::default() })
    }
    pub fn from_slice(device: Device, data: &[T]) -> Result<Self> {
        let mut ptr = std::ptr::null_mut();
        let bytes = std::mem::size_of_val(data);
        sys::check(unsafe { sys::ag_alloc(device.raw(), bytes, &mut ptr) })?;
        sys::check(unsafe { sys::ag_upload(device.raw(), ptr, data.as_ptr() as *const c_void, bytes) })?;
        // pageable memory: the copy has been staged when the call returns
        Ok(Self { device, ptr, len: data.len(), _marker: Default::default() })
    }
    pub fn to_vec(&self) -> Result<Vec<T>> {
        let mut out = Vec::<T>::with_capacity(self.len);
        let bytes = self.len * std::mem::size_of::<T>();
        sys::check(unsafe {
            sys::ag_download(self.device.raw(), out.as_mut_ptr() as *mut c_void, self.ptr, bytes)
        })?;
        unsafe { out.set_len(self.len) };
        Ok(out)
    }
    pub fn device_ptr(&self) -> *const c_void {
        self.ptr
    }
    pub fn device_ptr_mut(&mut self) -> *mut c_void {
        self.ptr
    }
    pub fn len(&self) -> usize {
        self.len
    }
}
impl<T> Drop for Buffer<T> {
    fn drop(&mut self) {
        unsafe { sys::ag_free(self.device.raw(), self.ptr) };
    }
}

/// f32 / bf16 -> the library's dtype code; everything else is `Dot unimplemented`.
pub fn dtype_code(scalar_type: autograph::krnl::scalar::ScalarType) -> Result<c_int> {
    use autograph::krnl::scalar::ScalarType::*;
    Ok(match scalar_type {
        F32 => sys::AG_F32,
        BF16 => sys::AG_BF16,
        other => bail!("Dot unimplemented for {other:?}!"),
    })
}

/// Replaces the `macro_wrap!` match with its kernel builder, split-k temporary and
/// `sum_axis_with` in `fn gemm` (src/tensor/linalg.rs:303-358).
#[allow(clippy::too_many_arguments)]
pub fn gemm(
    device: &Device, dtype: c_int, m: usize, k: usize, n: usize, alpha: f32,
    a: *const c_void, offset_a: usize, rsa: isize, csa: isize,
    b: *const c_void, offset_b: usize, rsb: isize, csb: isize,
    beta: f32, c: *mut c_void, offset_c: usize, rsc: isize, csc: isize,
) -> Result<()> {
    sys::check(unsafe {
        sys::ag_gemm(device.raw(), dtype, m as i64, k as i64, n as i64, alpha,
            a, offset_a as i64, rsa as i64, csa as i64,
            b, offset_b as i64, rsb as i64, csb as i64,
            beta, c, offset_c as i64, rsc as i64, csc as i64)
    })
}

/// Replaces the device blocks of `relu` / `relu_mut` (src/learn/neural_network/layer.rs:1315-1331,
/// 1352-1368); `y == x` is the in-place form.
pub fn relu(device: &Device, dtype: c_int, x: *const c_void, y: *mut c_void, len: usize) -> Result<()> {
    sys::check(unsafe { sys::ag_relu(device.raw(), dtype, x, y, len as i64) })
}

/// Replaces `relu_backward` / `relu_backward_mut` (layer.rs:1435-1458, 1483-1509).
pub fn relu_backward(device: &Device, dtype: c_int, x: *const c_void, dy: *const c_void,
                     dx: *mut c_void, len: usize) -> Result<()> {
    sys::check(unsafe { sys::ag_relu_backward(device.raw(), dtype, x, dy, dx, len as i64) })
}

/// Replaces the device block of `MaxPool2::max_pool2` (src/tensor/ops.rs:1117-1133).
#[allow(clippy::too_many_arguments)]
pub fn max_pool2(device: &Device, dtype: c_int, x: *const c_void, [bs, c, ih, iw]: [usize; 4],
                 size: [usize; 2], strides: [usize; 2], y: *mut c_void) -> Result<()> {
    sys::check(unsafe {
        sys::ag_max_pool2(device.raw(), dtype, x, bs as i64, c as i64, ih as i64, iw as i64,
            size[0] as i32, size[1] as i32, strides[0] as i32, strides[1] as i32, y)
    })
}

/// Replaces the device block of `MaxPool2Backward::max_pool2_backward` (ops.rs:1252-1264): the
/// gradient buffer arrives holding a copy of the forward input (layer.rs:1203-1212).
#[allow(clippy::too_many_arguments)]
pub fn max_pool2_backward(device: &Device, dtype: c_int, dx: *mut c_void, [bs, c, ih, iw]: [usize; 4],
                          size: [usize; 2], strides: [usize; 2], dy: *const c_void) -> Result<()> {
    sys::check(unsafe {
        sys::ag_max_pool2_backward(device.raw(), dtype, dx, bs as i64, c as i64, ih as i64, iw as i64,
            size[0] as i32, size[1] as i32, strides[0] as i32, strides[1] as i32, dy)
    })
}

fn conv_options(filter: [usize; 2], padding: [usize; 2], stride: [usize; 2], dilation: [usize; 2])
    -> sys::ag_conv2_options {
    let a = |v: [usize; 2]| [v[0] as i32, v[1] as i32];
    sys::ag_conv2_options { filter: a(filter), padding: a(padding), stride: a(stride), dilation: a(dilation) }
}

/// Replaces `conv2_im2col` forward: im2col -> dot -> permute to NCHW -> bias add
/// (layer.rs:950-1005, 944-946) with one implicit-GEMM call that writes NCHW.
#[allow(clippy::too_many_arguments)]
pub fn conv2_forward(device: &Device, dtype: c_int, x: *const c_void, [bs, ic, ih, iw]: [usize; 4],
                     w: *const c_void, oc: usize, bias: Option<*const c_void>,
                     filter: [usize; 2], padding: [usize; 2], stride: [usize; 2], dilation: [usize; 2],
                     fuse_relu: bool, y: *mut c_void) -> Result<()> {
    let opt = conv_options(filter, padding, stride, dilation);
    sys::check(unsafe {
        sys::ag_conv2_forward(device.raw(), dtype, x, bs as i64, ic as i64, ih as i64, iw as i64, w,
            oc as i64, bias.unwrap_or(std::ptr::null()), &opt, fuse_relu as c_int, y)
    })
}

/// The two backward edges of `conv2_im2col` (layer.rs:976-997).
#[allow(clippy::too_many_arguments)]
pub fn conv2_backward_input(device: &Device, dtype: c_int, w: *const c_void, oc: usize, ic: usize,
                            dy: *const c_void, bs: usize, ih: usize, iw: usize,
                            filter: [usize; 2], padding: [usize; 2], stride: [usize; 2],
                            dilation: [usize; 2], dx: *mut c_void) -> Result<()> {
    let opt = conv_options(filter, padding, stride, dilation);
    sys::check(unsafe {
        sys::ag_conv2_backward_input(device.raw(), dtype, w, oc as i64, ic as i64, dy, bs as i64,
            ih as i64, iw as i64, &opt, dx)
    })
}
#[allow(clippy::too_many_arguments)]
pub fn conv2_backward_weight(device: &Device, dtype: c_int, x: *const c_void, [bs, ic, ih, iw]: [usize; 4],
                             dy: *const c_void, oc: usize, filter: [usize; 2], padding: [usize; 2],
                             stride: [usize; 2], dilation: [usize; 2], accumulate: bool,
                             dw: *mut c_void) -> Result<()> {
    let opt = conv_options(filter, padding, stride, dilation);
    sys::check(unsafe {
        sys::ag_conv2_backward_weight(device.raw(), dtype, x, bs as i64, ic as i64, ih as i64, iw as i64,
            dy, oc as i64, &opt, if accumulate { 1.0 } else { 0.0 }, dw)
    })
}

/// Replaces cross_entropy_loss_device + sum (src/learn/criterion.rs:229-254): the summed loss as
/// a host f32 (synchronises, as the reference does).
pub fn cross_entropy_loss(device: &Device, dtype: c_int, label_dtype: c_int, x: *const c_void,
                          t: *const c_void, bs: usize, classes: usize) -> Result<f32> {
    let mut loss = 0f32;
    sys::check(unsafe {
        sys::ag_cross_entropy_loss(device.raw(), dtype, label_dtype, x, t, bs as i64, classes as i64, &mut loss)
    })?;
    Ok(loss)
}

/// Replaces the kernel dispatch of SGD with momentum (optimizer.rs:472-498).
#[allow(clippy::too_many_arguments)]
pub fn sgd_update_with_momentum(device: &Device, dtype: c_int, w: *mut c_void, g: *const c_void,
                                v: *mut c_void, len: usize, lr: f32, momentum: f32) -> Result<()> {
    sys::check(unsafe {
        sys::ag_sgd_update_momentum(device.raw(), dtype, w, g, v, len as i64, lr, momentum)
    })
}

/// Data-parallel training over the GPUs of one box (the reference has none): one communicator,
/// one fused call per rank and step (gradient all-reduce over NVLink + 1/world + SGD update).
pub struct Comm(*mut sys::ag_comm);
impl Comm {
    pub fn new(devices: &[Device]) -> Result<Self> {
        let raws: Vec<*mut sys::ag_device> = devices.iter().map(|d| d.raw()).collect();
        let mut out = std::ptr::null_mut();
        sys::check(unsafe { sys::ag_comm_create(raws.as_ptr(), raws.len() as c_int, &mut out) })?;
        Ok(Self(out))
    }
    pub fn allreduce_update(&self, model: *mut sys::ag_model, rank: usize, lr: f32) -> Result<()> {
        sys::check(unsafe { sys::ag_model_allreduce_update(model, self.0, rank as c_int, lr) })
    }
}
impl Drop for Comm {
    fn drop(&mut self) {
        unsafe { sys::ag_comm_destroy(self.0) };
    }
}
