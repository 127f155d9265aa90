//
// Test artifact written by hand for tests/test_mtrt_shim.py: x[i] += v for i < n.
// Parameters follow the launch convention for a statically shaped memref plus two scalars.
//
.version 8.0
.target sm_80
.address_size 64

.visible .entry add_scalar(
    .param .u64 add_scalar_param_0,
    .param .u32 add_scalar_param_1,
    .param .f32 add_scalar_param_2
)
{
    .reg .pred  %p<2>;
    .reg .b32   %r<6>;
    .reg .f32   %f<4>;
    .reg .b64   %rd<5>;

    ld.param.u64    %rd1, [add_scalar_param_0];
    ld.param.u32    %r1, [add_scalar_param_1];
    ld.param.f32    %f1, [add_scalar_param_2];
    mov.u32         %r2, %ctaid.x;
    mov.u32         %r3, %ntid.x;
    mov.u32         %r4, %tid.x;
    mad.lo.s32      %r5, %r2, %r3, %r4;
    setp.ge.s32     %p1, %r5, %r1;
    @%p1 bra        DONE;
    cvta.to.global.u64 %rd2, %rd1;
    mul.wide.s32    %rd3, %r5, 4;
    add.s64         %rd4, %rd2, %rd3;
    ld.global.f32   %f2, [%rd4];
    add.f32         %f3, %f2, %f1;
    st.global.f32   [%rd4], %f3;
DONE:
    ret;
}
