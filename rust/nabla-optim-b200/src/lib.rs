//! nabla-train's optimizers on B200: `Optimizer<f32, Cuda>` and `OptimState<f32, Cuda>`
//! (nabla-train/src/optim/core.rs:9-44, 64-79) implemented over libnabla_optim_b200.so.
//!
//! Each type owns one library handle.  A handle holds the optimizer state (m, v / velocity, fp32
//! masters) on the device; parameters and gradients stay nabla tensors and cross the boundary as
//! the address `Tensor::device_ptr()` returns (nabla-core/src/common/tensor/mod.rs:132-134) plus
//! `rows * cols`.  Work is enqueued on nabla's own stream, `cuda_compute_stream()`
//! (nabla-core/src/cuda_hip/cuda/core.rs:618-620), so it is ordered with the kernels that
//! produced the gradients.  There is no CPU fallback: without a CUDA device the constructors panic
//! with the library's message.
//!
//! Types: [`B200Sgd`], [`B200Adam`], [`B200AdamW`] (alg.rs:7-428), [`B200GroupOptimizer`]
//! (groups.rs:152-313), [`B200MixedAdamW`] (bf16 parameters and gradients, fp32 state; the
//! reference has no counterpart: its optimizers have one scalar type).

pub mod ffi;

use std::collections::HashMap;
use std::ffi::CStr;
use std::os::raw::c_void;

use nabla_core::backend::Cuda;
use nabla_core::tensor::Tensor;
use nabla_train::optim::core::{optim_kind_str, parse_optim_kind};
use nabla_train::optim::{OptimKind, OptimMeta, OptimState, Optimizer, ParamGroupConfig};

use ffi::*;

// ---------------------------------------------------------------------------------------------
// handle

/// One `nbo_optimizer`.  `Send` (one host thread drives it at a time), not `Sync`.
struct Handle {
    raw: *mut NboOptimizer,
}

unsafe impl Send for Handle {}

impl Handle {
    fn new() -> Self {
        let mut raw = std::ptr::null_mut();
        let stream = nabla_core::cuda_compute_stream().cu_stream() as *mut c_void;
        let rc = unsafe { nbo_create(0, stream, &mut raw) };
        if rc != NBO_OK {
            panic!("{}", last_error(std::ptr::null()));
        }
        Self { raw }
    }

    /// Misuse panics, as the reference's `assert_eq!`s do (alg.rs:110-119).
    fn check(&self, rc: i32) {
        if rc != NBO_OK {
            panic!("{}", last_error(self.raw));
        }
    }

    /// The `Result<(), String>` flavour `OptimState` wants.
    fn result(&self, rc: i32) -> Result<(), String> {
        if rc == NBO_OK { Ok(()) } else { Err(last_error(self.raw)) }
    }

    fn add_group(&self, cfg: &NboGroupConfig) -> i32 {
        let mut id = 0i32;
        self.check(unsafe { nbo_add_group(self.raw, cfg, &mut id) });
        id
    }

    fn set_tensors(&self, numel: &[u64], group_ids: Option<&[i32]>, precision: i32) {
        let gids = group_ids.map_or(std::ptr::null(), <[i32]>::as_ptr);
        self.check(unsafe { nbo_set_tensors(self.raw, numel.len() as u64, numel.as_ptr(), gids, precision) });
    }

    fn group(&self, gid: usize) -> NboGroupConfig {
        let mut cfg = NboGroupConfig::default();
        self.check(unsafe { nbo_get_group(self.raw, gid as i32, &mut cfg) });
        cfg
    }

    fn step_count(&self, gid: usize) -> usize {
        let mut c = 0u64;
        self.check(unsafe { nbo_step_count(self.raw, gid as i32, &mut c) });
        c as usize
    }

    /// State tensor `which` (0 = m / SGD velocity, 1 = v, 2 = fp32 master) of tensor `i`, with the
    /// parameter's own shape, as the reference keeps it (alg.rs:20-27).
    fn state(&self, i: usize, which: i32, shape: (usize, usize)) -> Tensor<f32, Cuda> {
        let mut host = vec![0f32; shape.0 * shape.1];
        self.check(unsafe { nbo_state_export(self.raw, i as u64, which, host.as_mut_ptr()) });
        Tensor::from_vec(host, shape.0, shape.1)
    }

    fn load_state(&self, i: usize, which: i32, t: &Tensor<f32, Cuda>, numel: usize, key: &str) -> Result<(), String> {
        let host = t.to_vec();
        if host.len() != numel {
            // what the reference's next step would trip over (tensor/ops.rs:638-646), reported at load time
            return Err(format!("nabla: axpy_inplace shapes must match ({key}: {:?} for {numel} elements)", t.shape()));
        }
        self.result(unsafe { nbo_state_import(self.raw, i as u64, which, host.as_ptr()) })
    }
}

impl Drop for Handle {
    fn drop(&mut self) {
        unsafe { nbo_destroy(self.raw) };
    }
}

fn last_error(h: *const NboOptimizer) -> String {
    unsafe { CStr::from_ptr(nbo_last_error(h)) }.to_string_lossy().into_owned()
}

fn kind_code(kind: OptimKind) -> i32 {
    match kind {
        OptimKind::AdamW => NBO_ADAMW,
        OptimKind::Adam => NBO_ADAM,
        OptimKind::Sgd => NBO_SGD,
    }
}

fn numel_of(shapes: &[(usize, usize)]) -> Vec<u64> {
    shapes.iter().map(|&(r, c)| (r * c) as u64).collect()
}

fn param_ptrs(params: &mut [&mut Tensor<f32, Cuda>]) -> Vec<*mut c_void> {
    params.iter().map(|t| t.device_ptr() as *mut c_void).collect()
}

fn grad_ptrs(grads: &[&Tensor<f32, Cuda>]) -> Vec<*const c_void> {
    grads.iter().map(|t| t.device_ptr() as *const c_void).collect()
}

/// `Optimizer::step` over the handle: the reference's two length assertions, then one call.
fn step_f32(h: &Handle, who: &str, n: usize, params: &mut [&mut Tensor<f32, Cuda>], grads: &[&Tensor<f32, Cuda>]) {
    assert_eq!(params.len(), grads.len(), "nabla-train: {who} params/grads length mismatch");
    assert_eq!(params.len(), n, "nabla-train: {who} params count mismatch");
    let p = param_ptrs(params);
    let g = grad_ptrs(grads);
    h.check(unsafe { nbo_step(h.raw, n as u64, p.as_ptr(), g.as_ptr()) });
}

/// m{i} / v{i} (or only v{i} for SGD) of a list of tensors, in the reference's order (alg.rs:476-485).
fn named_state(h: &Handle, shapes: &[(usize, usize)], idx: &[usize], sgd: bool) -> Vec<(String, Tensor<f32, Cuda>)> {
    let mut out = Vec::new();
    if !sgd {
        for (li, &i) in idx.iter().enumerate() {
            out.push((format!("m{li}"), h.state(i, 0, shapes[i])));
        }
    }
    for (li, &i) in idx.iter().enumerate() {
        out.push((format!("v{li}"), h.state(i, if sgd { 0 } else { 1 }, shapes[i])));
    }
    out
}

/// The reference's `load_state_tensors` (alg.rs:487-518, 620-640): keys `m{i}` / `v{i}`, every index required.
fn load_named_state(h: &Handle, shapes: &[(usize, usize)], idx: &[usize], sgd: bool,
                    tensors: &[(String, Tensor<f32, Cuda>)]) -> Result<(), String> {
    let mut m: Vec<Option<&Tensor<f32, Cuda>>> = vec![None; idx.len()];
    let mut v: Vec<Option<&Tensor<f32, Cuda>>> = vec![None; idx.len()];
    for (name, t) in tensors {
        if let Some(rest) = name.strip_prefix('m') {
            if sgd { continue; }
            let i = rest.parse::<usize>().map_err(|_| format!("bad tensor key: {name}"))?;
            if i >= m.len() { return Err(format!("m index out of range: {i}")); }
            m[i] = Some(t);
        } else if let Some(rest) = name.strip_prefix('v') {
            let i = rest.parse::<usize>().map_err(|_| format!("bad tensor key: {name}"))?;
            if i >= v.len() { return Err(format!("v index out of range: {i}")); }
            v[i] = Some(t);
        }
    }
    if !sgd {
        for (li, t) in m.iter().enumerate() {
            let t = t.ok_or_else(|| format!("missing m{li}"))?;
            let (r, c) = shapes[idx[li]];
            h.load_state(idx[li], 0, t, r * c, &format!("m{li}"))?;
        }
    }
    for (li, t) in v.iter().enumerate() {
        let t = t.ok_or_else(|| format!("missing v{li}"))?;
        let (r, c) = shapes[idx[li]];
        h.load_state(idx[li], if sgd { 0 } else { 1 }, t, r * c, &format!("v{li}"))?;
    }
    Ok(())
}

fn meta_of(h: &Handle, gid: usize) -> OptimMeta {
    let c = h.group(gid);
    let kind = match c.kind { NBO_ADAM => OptimKind::Adam, NBO_SGD => OptimKind::Sgd, _ => OptimKind::AdamW };
    let adamish = c.kind != NBO_SGD;
    OptimMeta {
        kind,
        lr: c.lr,
        beta1: if adamish { c.beta1 } else { 0.0 },
        beta2: if adamish { c.beta2 } else { 0.0 },
        eps: if adamish { c.eps } else { 0.0 },
        weight_decay: if c.kind == NBO_ADAM { 0.0 } else { c.weight_decay },
        momentum: if adamish { 0.0 } else { c.momentum },
        step_count: if adamish { h.step_count(gid) } else { 0 },
    }
}

/// `load_meta` of the three optimizers (alg.rs:534-556, 594-615, 657-671): the kind must match.
fn load_meta_into(h: &Handle, gid: usize, meta: &OptimMeta) -> Result<(), String> {
    let mut c = h.group(gid);
    if kind_code(meta.kind) != c.kind {
        return Err("optim kind mismatch".to_owned());
    }
    c.lr = meta.lr;
    if c.kind == NBO_SGD {
        c.momentum = meta.momentum;
        c.weight_decay = meta.weight_decay;
    } else {
        c.beta1 = meta.beta1;
        c.beta2 = meta.beta2;
        c.eps = meta.eps;
        if c.kind == NBO_ADAMW {
            c.weight_decay = meta.weight_decay;
        }
    }
    h.result(unsafe { nbo_set_group(h.raw, gid as i32, &c) })?;
    if c.kind != NBO_SGD {
        h.result(unsafe { nbo_set_step_count(h.raw, gid as i32, meta.step_count as u64) })?;
    }
    Ok(())
}

// ---------------------------------------------------------------------------------------------
// Sgd / Adam / AdamW

macro_rules! single_group_optimizer {
    ($name:ident, $who:literal, $kind:expr, $optkind:expr, $sgd:expr, $doc:literal) => {
        #[doc = $doc]
        pub struct $name {
            h: Handle,
            shapes: Vec<(usize, usize)>,
        }

        impl $name {
            fn with_config(cfg: NboGroupConfig, param_shapes: &[(usize, usize)]) -> Self {
                let h = Handle::new();
                h.add_group(&cfg);
                h.set_tensors(&numel_of(param_shapes), None, NBO_F32);
                Self { h, shapes: param_shapes.to_vec() }
            }

            #[must_use]
            pub fn from_params(lr: f64, params: &[&Tensor<f32, Cuda>]) -> Self {
                let shapes: Vec<(usize, usize)> = params.iter().map(|p| p.shape()).collect();
                Self::new(lr, &shapes)
            }

            fn update(&mut self, f: impl FnOnce(&mut NboGroupConfig)) {
                let mut c = self.h.group(0);
                f(&mut c);
                self.h.check(unsafe { nbo_set_group(self.h.raw, 0, &c) });
            }

            #[must_use]
            pub fn lr(&self) -> f64 {
                self.h.group(0).lr
            }

            /// Every gradient of the list becomes zeros on the device (the free function `zero_grad`,
            /// nabla-ml/src/autograd/ops.rs:1668-1673, without the reallocation).
            pub fn zero_grad(&mut self, grads: &mut [&mut Tensor<f32, Cuda>]) {
                assert_eq!(grads.len(), self.shapes.len(), concat!("nabla-train: ", $who, " params count mismatch"));
                let g = param_ptrs(grads);
                self.h.check(unsafe { nbo_zero_grad(self.h.raw, g.len() as u64, g.as_ptr()) });
            }
        }

        impl Optimizer<f32, Cuda> for $name {
            fn step(&mut self, params: &mut [&mut Tensor<f32, Cuda>], grads: &[&Tensor<f32, Cuda>]) {
                step_f32(&self.h, $who, self.shapes.len(), params, grads);
            }

            fn reset(&mut self) {
                self.h.check(unsafe { nbo_reset(self.h.raw) });
            }

            fn set_lr(&mut self, lr: f64) {
                self.h.check(unsafe { nbo_set_lr(self.h.raw, lr) });
            }
        }

        impl OptimState<f32, Cuda> for $name {
            fn kind(&self) -> OptimKind {
                $optkind
            }

            fn state_tensors(&self) -> Vec<(String, Tensor<f32, Cuda>)> {
                let idx: Vec<usize> = (0..self.shapes.len()).collect();
                named_state(&self.h, &self.shapes, &idx, $sgd)
            }

            fn load_state_tensors(&mut self, tensors: &[(String, Tensor<f32, Cuda>)]) -> Result<(), String> {
                let idx: Vec<usize> = (0..self.shapes.len()).collect();
                load_named_state(&self.h, &self.shapes, &idx, $sgd, tensors)
            }

            fn meta(&self) -> OptimMeta {
                meta_of(&self.h, 0)
            }

            fn load_meta(&mut self, meta: &OptimMeta) -> Result<(), String> {
                load_meta_into(&self.h, 0, meta)
            }
        }
    };
}

single_group_optimizer!(B200Sgd, "Sgd", NBO_SGD, OptimKind::Sgd, true,
    "`Sgd<f32, Cuda>` (alg.rs:310-428): plain, weight decay, momentum; one kernel launch per step.");
single_group_optimizer!(B200Adam, "Adam", NBO_ADAM, OptimKind::Adam, false,
    "`Adam<f32, Cuda>` (alg.rs:169-308); one kernel launch per step whatever the tensor count.");
single_group_optimizer!(B200AdamW, "AdamW", NBO_ADAMW, OptimKind::AdamW, false,
    "`AdamW<f32, Cuda>` (alg.rs:7-167): decoupled decay applied before the update is subtracted.");

impl B200Sgd {
    /// `Sgd::new` (alg.rs:319-331): momentum 0, weight decay 0.
    #[must_use]
    pub fn new(lr: f64, param_shapes: &[(usize, usize)]) -> Self {
        Self::with_config(NboGroupConfig { kind: NBO_SGD, lr, ..Default::default() }, param_shapes)
    }
    #[must_use]
    pub fn momentum(mut self, m: f64) -> Self {
        self.update(|c| c.momentum = m);
        self
    }
    #[must_use]
    pub fn weight_decay(mut self, wd: f64) -> Self {
        self.update(|c| c.weight_decay = wd);
        self
    }
}

impl B200Adam {
    /// `Adam::new` (alg.rs:181-201): betas 0.9 / 0.999, eps 1e-8.
    #[must_use]
    pub fn new(lr: f64, param_shapes: &[(usize, usize)]) -> Self {
        Self::with_config(
            NboGroupConfig { kind: NBO_ADAM, lr, beta1: 0.9, beta2: 0.999, eps: 1e-8, ..Default::default() },
            param_shapes,
        )
    }
    #[must_use]
    pub fn betas(mut self, b1: f64, b2: f64) -> Self {
        self.update(|c| { c.beta1 = b1; c.beta2 = b2; });
        self
    }
    #[must_use]
    pub fn eps(mut self, eps: f64) -> Self {
        self.update(|c| c.eps = eps);
        self
    }
    #[must_use]
    pub fn step_count(&self) -> usize {
        self.h.step_count(0)
    }
}

impl B200AdamW {
    /// `AdamW::new` (alg.rs:20-40): betas 0.9 / 0.999, eps 1e-8, weight decay 0.01.
    #[must_use]
    pub fn new(lr: f64, param_shapes: &[(usize, usize)]) -> Self {
        Self::with_config(
            NboGroupConfig { kind: NBO_ADAMW, lr, beta1: 0.9, beta2: 0.999, eps: 1e-8, weight_decay: 0.01, momentum: 0.0 },
            param_shapes,
        )
    }
    #[must_use]
    pub fn betas(mut self, b1: f64, b2: f64) -> Self {
        self.update(|c| { c.beta1 = b1; c.beta2 = b2; });
        self
    }
    #[must_use]
    pub fn eps(mut self, eps: f64) -> Self {
        self.update(|c| c.eps = eps);
        self
    }
    #[must_use]
    pub fn weight_decay(mut self, wd: f64) -> Self {
        self.update(|c| c.weight_decay = wd);
        self
    }
    #[must_use]
    pub fn step_count(&self) -> usize {
        self.h.step_count(0)
    }
}

// ---------------------------------------------------------------------------------------------
// GroupOptimizer

/// `GroupOptimizer<f32, Cuda>` (groups.rs:152-313).  The reference clones every member tensor into a
/// per-group optimizer and back on each step; here a group is a hyper-parameter set plus a range
/// of the device-resident chunk list, and a step is one launch per non-empty group.
pub struct B200GroupOptimizer {
    h: Handle,
    shapes: Vec<(usize, usize)>,
    /// per kept group: (name, kind, member tensor indices in list order)
    groups: Vec<(String, OptimKind, Vec<usize>)>,
}

fn group_config_c(cfg: &ParamGroupConfig) -> NboGroupConfig {
    NboGroupConfig {
        kind: kind_code(cfg.kind),
        lr: cfg.lr,
        beta1: cfg.beta1,
        beta2: cfg.beta2,
        eps: cfg.eps,
        weight_decay: cfg.weight_decay,
        momentum: cfg.momentum,
    }
}

/// The routing of `from_named_params` (groups.rs:168-226): first matching group wins, the rest goes to the
/// default group, an unassigned tensor is an error, empty groups are dropped.
fn assign_groups(names: &[&str], groups: &[ParamGroupConfig], default_group: Option<ParamGroupConfig>)
                 -> Result<Vec<(ParamGroupConfig, Vec<usize>)>, String> {
    let mut buckets: Vec<(ParamGroupConfig, Vec<usize>)> = groups.iter().cloned().map(|c| (c, Vec::new())).collect();
    let mut default_bucket = default_group.map(|c| (c, Vec::new()));
    for (i, name) in names.iter().enumerate() {
        let mut placed = false;
        for (cfg, idxs) in buckets.iter_mut() {
            if cfg.selector.matches(name) {
                idxs.push(i);
                placed = true;
                break;
            }
        }
        if !placed {
            match default_bucket.as_mut() {
                Some((_, idxs)) => idxs.push(i),
                None => return Err("nabla-train: group assignment incomplete".to_owned()),
            }
        }
    }
    let mut kept: Vec<(ParamGroupConfig, Vec<usize>)> = buckets.into_iter().filter(|(_, i)| !i.is_empty()).collect();
    if let Some(b) = default_bucket {
        if !b.1.is_empty() {
            kept.push(b);
        }
    }
    Ok(kept)
}

impl B200GroupOptimizer {
    pub fn from_named_params(named: &[(&str, &Tensor<f32, Cuda>)], groups: &[ParamGroupConfig],
                             default_group: Option<ParamGroupConfig>) -> Result<Self, String> {
        let names: Vec<&str> = named.iter().map(|(n, _)| *n).collect();
        let shapes: Vec<(usize, usize)> = named.iter().map(|(_, t)| t.shape()).collect();
        let kept = assign_groups(&names, groups, default_group)?;
        let h = Handle::new();
        let mut gid_of = vec![0i32; named.len()];
        let mut meta = Vec::new();
        for (cfg, idxs) in &kept {
            let gid = h.add_group(&group_config_c(cfg));
            for &i in idxs {
                gid_of[i] = gid;
            }
            meta.push((cfg.name.clone(), cfg.kind, idxs.clone()));
        }
        h.set_tensors(&numel_of(&shapes), Some(&gid_of), NBO_F32);
        Ok(Self { h, shapes, groups: meta })
    }

    #[must_use]
    pub fn groups(&self) -> usize {
        self.groups.len()
    }

    pub fn zero_grad(&mut self, grads: &mut [&mut Tensor<f32, Cuda>]) {
        assert_eq!(grads.len(), self.shapes.len(), "nabla-train: GroupOptimizer params count mismatch");
        let g = param_ptrs(grads);
        self.h.check(unsafe { nbo_zero_grad(self.h.raw, g.len() as u64, g.as_ptr()) });
    }
}

impl Optimizer<f32, Cuda> for B200GroupOptimizer {
    fn step(&mut self, params: &mut [&mut Tensor<f32, Cuda>], grads: &[&Tensor<f32, Cuda>]) {
        step_f32(&self.h, "GroupOptimizer", self.shapes.len(), params, grads);
    }

    fn reset(&mut self) {
        self.h.check(unsafe { nbo_reset(self.h.raw) });
    }

    /// Group k gets `base_lr[k] * lr / base_lr[0]`, or `lr` when `base_lr[0] <= 0` (groups.rs:301-312);
    /// the library applies the same rule.
    fn set_lr(&mut self, lr: f64) {
        self.h.check(unsafe { nbo_set_lr(self.h.raw, lr) });
    }
}

impl OptimState<f32, Cuda> for B200GroupOptimizer {
    fn kind(&self) -> OptimKind {
        OptimKind::AdamW
    }

    fn state_tensors(&self) -> Vec<(String, Tensor<f32, Cuda>)> {
        let mut out = Vec::new();
        for (gi, (_, kind, idx)) in self.groups.iter().enumerate() {
            for (name, t) in named_state(&self.h, &self.shapes, idx, matches!(kind, OptimKind::Sgd)) {
                out.push((format!("g{gi}.{name}"), t));
            }
        }
        out
    }

    fn load_state_tensors(&mut self, tensors: &[(String, Tensor<f32, Cuda>)]) -> Result<(), String> {
        let mut buckets: Vec<Vec<(String, Tensor<f32, Cuda>)>> = vec![Vec::new(); self.groups.len()];
        for (name, t) in tensors {
            let (g, rest) = name.split_once('.').ok_or_else(|| format!("bad group tensor key: {name}"))?;
            let idx = g.strip_prefix('g').ok_or_else(|| format!("bad group tensor key: {name}"))?;
            let gi = idx.parse::<usize>().map_err(|_| format!("bad group index: {idx}"))?;
            if gi >= buckets.len() {
                return Err(format!("group index out of range: {gi}"));
            }
            buckets[gi].push((rest.to_owned(), t.clone()));
        }
        for (gi, (_, kind, idx)) in self.groups.iter().enumerate() {
            load_named_state(&self.h, &self.shapes, idx, matches!(kind, OptimKind::Sgd), &buckets[gi])?;
        }
        Ok(())
    }

    fn meta(&self) -> OptimMeta {
        // groups.rs:355-366: only the base learning rate is meaningful at this level
        OptimMeta { kind: OptimKind::AdamW, lr: self.h.group(0).lr, beta1: 0.0, beta2: 0.0, eps: 0.0,
                    weight_decay: 0.0, momentum: 0.0, step_count: 0 }
    }

    fn load_meta(&mut self, _meta: &OptimMeta) -> Result<(), String> {
        Ok(())
    }

    fn meta_pairs(&self) -> Vec<(String, String)> {
        let mut out = vec![("optim.group.count".to_owned(), self.groups.len().to_string())];
        for (gi, (name, _, _)) in self.groups.iter().enumerate() {
            out.push((format!("optim.group.{gi}.name"), name.clone()));
            let m = meta_of(&self.h, gi);
            out.push((format!("optim.group.{gi}.kind"), optim_kind_str(m.kind)));
            out.push((format!("optim.group.{gi}.lr"), m.lr.to_string()));
            out.push((format!("optim.group.{gi}.beta1"), m.beta1.to_string()));
            out.push((format!("optim.group.{gi}.beta2"), m.beta2.to_string()));
            out.push((format!("optim.group.{gi}.eps"), m.eps.to_string()));
            out.push((format!("optim.group.{gi}.weight_decay"), m.weight_decay.to_string()));
            out.push((format!("optim.group.{gi}.momentum"), m.momentum.to_string()));
            out.push((format!("optim.group.{gi}.step_count"), m.step_count.to_string()));
        }
        out
    }

    fn load_meta_pairs(&mut self, map: &HashMap<String, String>) -> Result<(), String> {
        let get = |k: &str| map.get(k).map(String::as_str).ok_or_else(|| format!("missing {k}"));
        let num = |k: &str| -> Result<f64, String> {
            let v = get(k)?;
            v.parse::<f64>().map_err(|_| format!("bad {k}: {v}"))
        };
        let count = get("optim.group.count")?;
        let count = count.parse::<usize>().map_err(|_| format!("bad optim.group.count: {count}"))?;
        if count != self.groups.len() {
            return Err("optim.group.count mismatch".to_owned());
        }
        for gi in 0..self.groups.len() {
            if get(&format!("optim.group.{gi}.name"))? != self.groups[gi].0 {
                return Err(format!("optim.group.{gi}.name mismatch"));
            }
            let steps = get(&format!("optim.group.{gi}.step_count"))?;
            let meta = OptimMeta {
                kind: parse_optim_kind(get(&format!("optim.group.{gi}.kind"))?)?,
                lr: num(&format!("optim.group.{gi}.lr"))?,
                beta1: num(&format!("optim.group.{gi}.beta1"))?,
                beta2: num(&format!("optim.group.{gi}.beta2"))?,
                eps: num(&format!("optim.group.{gi}.eps"))?,
                weight_decay: num(&format!("optim.group.{gi}.weight_decay"))?,
                momentum: num(&format!("optim.group.{gi}.momentum"))?,
                step_count: steps.parse::<usize>().map_err(|_| format!("bad optim.group.{gi}.step_count: {steps}"))?,
            };
            load_meta_into(&self.h, gi, &meta)?;
        }
        Ok(())
    }
}

// ---------------------------------------------------------------------------------------------
// mixed precision

/// Outcome of one mixed-precision step.
#[derive(Clone, Copy, Debug)]
pub struct StepOutcome {
    /// false = skipped because a gradient was inf / NaN (trainer.rs:230-237)
    pub applied: bool,
    /// pre-clip global L2 norm of the unscaled gradients (0 when clipping is off)
    pub grad_norm: f64,
    /// the loss scale to use for the next backward pass
    pub loss_scale: f64,
    pub step_count: usize,
}

/// Mixed-precision Adam / AdamW: bf16 parameters and gradients owned by the caller, fp32 master / m / v
/// owned by the handle.  One `step_mixed` is the tail of `Trainer::train_epoch_with_max_steps`
/// (trainer.rs:230-283) in one call: `GradScaler::unscale_and_update` -> non-finite skip ->
/// `clip_grad_norm` -> AdamW on the masters -> bf16 parameters.
pub struct B200MixedAdamW {
    h: Handle,
    shapes: Vec<(usize, usize)>,
}

impl B200MixedAdamW {
    #[must_use]
    pub fn new(lr: f64, weight_decay: f64, param_shapes: &[(usize, usize)]) -> Self {
        let h = Handle::new();
        h.add_group(&NboGroupConfig { kind: NBO_ADAMW, lr, beta1: 0.9, beta2: 0.999, eps: 1e-8, weight_decay, momentum: 0.0 });
        h.set_tensors(&numel_of(param_shapes), None, NBO_MIXED_BF16);
        Self { h, shapes: param_shapes.to_vec() }
    }

    /// Seeds the fp32 masters from the bf16 parameters (exact widening).  `params[i]` is the device
    /// address of tensor i's bf16 storage (`Tensor::<bf16, Cuda>::device_ptr()`).
    pub fn init_master_from_params(&mut self, params: &[u64]) {
        assert_eq!(params.len(), self.shapes.len(), "nabla-train: AdamW params count mismatch");
        let p: Vec<*const c_void> = params.iter().map(|&a| a as *const c_void).collect();
        self.h.check(unsafe { nbo_init_master_from_params(self.h.raw, p.len() as u64, p.as_ptr()) });
    }

    /// One fused step on bf16 device tensors given by address.
    pub fn step_mixed(&mut self, params: &[u64], grads: &[u64], use_scaler: bool, max_norm: f64) -> StepOutcome {
        assert_eq!(params.len(), grads.len(), "nabla-train: AdamW params/grads length mismatch");
        assert_eq!(params.len(), self.shapes.len(), "nabla-train: AdamW params count mismatch");
        let p: Vec<*mut c_void> = params.iter().map(|&a| a as *mut c_void).collect();
        let g: Vec<*const c_void> = grads.iter().map(|&a| a as *const c_void).collect();
        let mut r = NboStepResult::default();
        self.h.check(unsafe {
            nbo_step_mixed(self.h.raw, p.len() as u64, p.as_ptr(), g.as_ptr(), use_scaler as i32, max_norm, &mut r)
        });
        StepOutcome { applied: r.applied != 0, grad_norm: r.grad_norm, loss_scale: r.loss_scale, step_count: r.step_count as usize }
    }

    pub fn zero_grad(&mut self, grads: &[u64]) {
        assert_eq!(grads.len(), self.shapes.len(), "nabla-train: AdamW params count mismatch");
        let g: Vec<*mut c_void> = grads.iter().map(|&a| a as *mut c_void).collect();
        self.h.check(unsafe { nbo_zero_grad(self.h.raw, g.len() as u64, g.as_ptr()) });
    }

    pub fn set_lr(&mut self, lr: f64) {
        self.h.check(unsafe { nbo_set_lr(self.h.raw, lr) });
    }

    pub fn reset(&mut self) {
        self.h.check(unsafe { nbo_reset(self.h.raw) });
    }

    /// `GradScaler::state` / `load_state` (core.rs:390-413): the scaler lives in the handle.
    #[must_use]
    pub fn scaler_state(&self) -> NboScalerState {
        let mut s = NboScalerState::default();
        self.h.check(unsafe { nbo_scaler_get(self.h.raw, &mut s) });
        s
    }

    pub fn load_scaler_state(&mut self, s: &NboScalerState) {
        self.h.check(unsafe { nbo_scaler_set(self.h.raw, s) });
    }
}

impl OptimState<f32, Cuda> for B200MixedAdamW {
    fn kind(&self) -> OptimKind {
        OptimKind::AdamW
    }

    /// m{i}, v{i} as the reference names them, plus the fp32 masters as w{i}; the reference's loaders skip
    /// names that start with neither `m` nor `v` (alg.rs:491-507).
    fn state_tensors(&self) -> Vec<(String, Tensor<f32, Cuda>)> {
        let idx: Vec<usize> = (0..self.shapes.len()).collect();
        let mut out = named_state(&self.h, &self.shapes, &idx, false);
        for &i in &idx {
            out.push((format!("w{i}"), self.h.state(i, 2, self.shapes[i])));
        }
        out
    }

    fn load_state_tensors(&mut self, tensors: &[(String, Tensor<f32, Cuda>)]) -> Result<(), String> {
        let idx: Vec<usize> = (0..self.shapes.len()).collect();
        load_named_state(&self.h, &self.shapes, &idx, false, tensors)?;
        for (name, t) in tensors {
            if let Some(rest) = name.strip_prefix('w') {
                let i = rest.parse::<usize>().map_err(|_| format!("bad tensor key: {name}"))?;
                if i >= self.shapes.len() {
                    return Err(format!("w index out of range: {i}"));
                }
                let (r, c) = self.shapes[i];
                self.h.load_state(i, 2, t, r * c, name)?;
            }
        }
        Ok(())
    }

    fn meta(&self) -> OptimMeta {
        meta_of(&self.h, 0)
    }

    fn load_meta(&mut self, meta: &OptimMeta) -> Result<(), String> {
        load_meta_into(&self.h, 0, meta)
    }
}
