package neureka.backend.cuda;

import neureka.Tensor;
import neureka.backend.api.BackendExtension;
import neureka.backend.api.ExecutionCall;
import neureka.backend.api.Extensions;
import neureka.backend.api.ImplementationFor;
import neureka.backend.api.ini.BackendLoader;
import neureka.backend.api.ini.ReceiveForDevice;
import neureka.backend.main.algorithms.*;
import neureka.backend.main.implementations.fun.api.ScalarFun;
import neureka.backend.main.operations.functions.*;
import neureka.backend.main.operations.linear.Convolution;
import neureka.backend.main.operations.linear.XConvLeft;
import neureka.backend.main.operations.linear.XConvRight;
import neureka.backend.main.operations.operator.*;
import neureka.backend.main.operations.other.AssignLeft;
import neureka.backend.main.operations.other.Sum;
import neureka.devices.cuda.CudaDevice;
import neureka.devices.cuda.CudaKernels;
import neureka.math.args.Arg;

import java.util.ArrayList;
import java.util.List;

/**
 *  BackendExtension that puts a CUDA ImplementationFor on every (Operation, Algorithm) pair of the convolution /
 *  broadcast / elementwise path -- the pair list of CLBackend._load (backend/ocl/CLBackend.java:200-325) minus
 *  DotProduct / Randomization. Install with {@code Neureka.get().backend().set(new CudaBackend())}
 *  (BackendContext.java:289-321); Tensor.of(...), Function.of("i0 x i1") and backward() then run unchanged on
 *  tensors moved to a CudaDevice. The executable twin is neureka_b200/backend.py. COMPILE-UNVERIFIED.
 */
public final class CudaBackend implements BackendExtension
{
    private final List<CudaDevice> _devices = new ArrayList<>();

    /** One CudaDevice per visible GPU; all of them are members of one native device group (nk_group_open: peer access
     *  between the members is enabled once), so that CudaKernels.convSharded can cut a large convolution across them. */
    public CudaBackend() {
        int n = CudaDevice.count();
        for ( int i = 0; i < Math.max(n, 1); i++ ) _devices.add(new CudaDevice(i));
    }

    /** "cuda" / "gpu" / "nvidia" / "first" / "b200" -> the first GPU; "cuda:2", "gpu:2" or a plain "2" -> that ordinal
     *  (the keyword scheme Device.get uses for OpenCL devices, devices/Query.java:22-24). */
    @Override public DeviceOption find( String key ) {
        String k = key.trim().toLowerCase();
        int ordinal = -1;
        if ( k.equals("cuda") || k.equals("gpu") || k.equals("nvidia") || k.equals("first") || k.equals("b200") ) ordinal = 0;
        else {
            String digits = k.startsWith("cuda:") || k.startsWith("gpu:") ? k.substring(k.indexOf(':') + 1) : k;
            if ( !digits.isEmpty() && digits.chars().allMatch(Character::isDigit) ) ordinal = Integer.parseInt(digits);
        }
        if ( ordinal >= 0 && ordinal < _devices.size() ) return new DeviceOption(_devices.get(ordinal), 1.0);
        return new DeviceOption(null, 0.0);
    }

    /** The devices of this backend, in ordinal order (the members of the native group). */
    public List<CudaDevice> devices() { return java.util.Collections.unmodifiableList(_devices); }

    @Override public void dispose() { _devices.forEach(CudaDevice::dispose); _devices.clear(); }
    @Override public boolean update( OwnerChangeRequest<Extensions> changeRequest ) { return true; }
    @Override public BackendLoader getLoader() { return receiver -> _load(receiver.forDevice(CudaDevice.class)); }

    private static int d( ExecutionCall<CudaDevice> call ) { return call.getValOf(Arg.DerivIdx.class); }

    private void _load( ReceiveForDevice<CudaDevice> receive )
    {
        Class[] operators = { Power.class, Addition.class, Subtraction.class, Multiplication.class, Division.class, Modulo.class };
        int[]   opCodes   = { 5, 0, 1, 2, 3, 4 };   // NK_OP_POW, ADD, SUB, MUL, DIV, MOD
        for ( int i = 0; i < operators.length; i++ ) {
            final int op = opCodes[i];
            receive.forOperation( operators[i] )
                   .set( BiScalarBroadcast.class, ctx -> (ImplementationFor<CudaDevice>) call -> CudaKernels.scalarBinary(op, call, d(call)) )
                   .set( Broadcast.class,         ctx -> (ImplementationFor<CudaDevice>) call -> CudaKernels.broadcast(op, call, d(call)) )
                   .set( BiElementwise.class,     ctx -> (ImplementationFor<CudaDevice>) call -> CudaKernels.binary(op, call, d(call)) );
        }
        receive.forOperation( AssignLeft.class )
               .set( BiScalarBroadcast.class,    ctx -> (ImplementationFor<CudaDevice>) call -> CudaKernels.scalarBinary(6, call, -1) )
               .set( ElementwiseAlgorithm.class, ctx -> (ImplementationFor<CudaDevice>) call -> CudaKernels.unary("idy", call, -1) );

        for ( Class conv : new Class[]{ Convolution.class, XConvLeft.class, XConvRight.class } )
            receive.forOperation( conv ).set( NDConvolution.class, ctx -> (ImplementationFor<CudaDevice>) call -> CudaKernels.conv(call, d(call)) );

        receive.forOperation( Sum.class ).set( SumAlgorithm.class, ctx -> (ImplementationFor<CudaDevice>) CudaKernels::sum );
        // a @ b is the convolution [M,K,1] x [1,K,N] -> [M,1,N] on padded views of the three matrices (no copy)
        receive.forOperation( neureka.backend.main.operations.linear.MatMul.class )
               .set( neureka.backend.main.algorithms.MatMulAlgorithm.class, ctx -> (ImplementationFor<CudaDevice>) CudaKernels::matMul );

        Object[][] activations = {
            { Absolute.class, ScalarFun.ABSOLUTE }, { Cosinus.class, ScalarFun.COSINUS }, { GaSU.class, ScalarFun.GASU }, { GaTU.class, ScalarFun.GATU },
            { Gaussian.class, ScalarFun.GAUSSIAN }, { GaussianFast.class, ScalarFun.GAUSSIAN_FAST }, { GeLU.class, ScalarFun.GELU },
            { Identity.class, ScalarFun.IDENTITY }, { Logarithm.class, ScalarFun.LOGARITHM }, { Quadratic.class, ScalarFun.QUADRATIC },
            { ReLU.class, ScalarFun.RELU }, { SeLU.class, ScalarFun.SELU }, { Sigmoid.class, ScalarFun.SIGMOID }, { SiLU.class, ScalarFun.SILU },
            { Sinus.class, ScalarFun.SINUS }, { Softplus.class, ScalarFun.SOFTPLUS }, { Softsign.class, ScalarFun.SOFTSIGN }, { Tanh.class, ScalarFun.TANH },
            { TanhFast.class, ScalarFun.TANH_FAST }, { Exp.class, ScalarFun.EXP }, { Cbrt.class, ScalarFun.CBRT }, { Log10.class, ScalarFun.LOG10 },
            { Sqrt.class, ScalarFun.SQRT }
        };
        for ( Object[] a : activations ) {
            final String id = ((ScalarFun) a[1]).id();
            receive.forOperation( (Class) a[0] )
                   .set( ElementwiseAlgorithm.class, ctx -> (ImplementationFor<CudaDevice>) call -> CudaKernels.unary(id, call, d(call)) )
                   .set( ScalarAlgorithm.class,      ctx -> (ImplementationFor<CudaDevice>) call -> CudaKernels.fillFun(id, call, d(call)) );
        }
    }
}
