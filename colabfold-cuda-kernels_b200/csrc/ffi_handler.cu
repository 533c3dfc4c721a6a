// The XLA FFI target `MkSample`: a thin wrapper that unpacks the call frame and forwards to the
// plain C entry point cck_mk_sample. Compiled only when CCK_FFI is defined and the XLA FFI headers
// are on the include path (they ship with jax; this repository does not carry them).
//
// Same binding as the reference's handler (src/diffusion/host.cuh:505-549): the platform stream,
// 1 + 74 untyped argument buffers (ext first), two results (positions, workspace) and the int32
// attributes samples, nsteps, flags; command-buffer compatible because nothing synchronises.
#ifdef CCK_FFI
#include <cuda_runtime.h>

#include "../../include/cck_b200.h"
#include "xla/ffi/api/ffi.h"

namespace ffi = xla::ffi;

static ffi::Error mk_sample_ffi(cudaStream_t stream, ffi::RemainingArgs args, ffi::Result<ffi::AnyBuffer> out,
                                ffi::Result<ffi::AnyBuffer> ws, int32_t samples, int32_t nsteps, int32_t flags) {
    if (args.size() != CCK_NUM_INPUTS + 1) {
        return ffi::Error(ffi::ErrorCode::kInvalidArgument, "MkSample: wrong number of inputs");
    }
    auto ext = args.get<ffi::AnyBuffer>(0);
    if (ext.has_error()) {
        return ext.error();
    }
    const void* in[CCK_NUM_INPUTS];
    size_t bytes[CCK_NUM_INPUTS];
    for (int i = 0; i < CCK_NUM_INPUTS; i++) {
        auto buf = args.get<ffi::AnyBuffer>(i + 1);
        if (buf.has_error()) {
            return buf.error();
        }
        in[i] = buf->untyped_data();
        bytes[i] = buf->size_bytes();
    }
    const int rc = cck_mk_sample(stream, static_cast<const int*>(ext->untyped_data()), in, bytes, CCK_NUM_INPUTS,
                                 static_cast<float*>(out->untyped_data()), int(out->dimensions()[1]),
                                 ws->untyped_data(), ws->size_bytes(), samples, nsteps, flags);
    if (rc == CCK_OK) {
        return ffi::Error::Success();
    }
    return ffi::Error(rc == CCK_E_LAUNCH || rc == CCK_E_DEVICE ? ffi::ErrorCode::kInternal : ffi::ErrorCode::kInvalidArgument,
                      cck_last_error());
}

XLA_FFI_DEFINE_HANDLER_SYMBOL(MkSample, mk_sample_ffi,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .RemainingArgs()
                                  .Ret<ffi::AnyBuffer>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int32_t>("samples")
                                  .Attr<int32_t>("nsteps")
                                  .Attr<int32_t>("flags"),
                              {ffi::Traits::kCmdBufferCompatible});
#endif
