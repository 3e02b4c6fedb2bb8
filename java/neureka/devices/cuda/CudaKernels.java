package neureka.devices.cuda;

import neureka.Tensor;
import neureka.backend.api.ExecutionCall;

import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;
import java.util.Arrays;
import java.util.List;

/**
 *  One static method per kernel entry point: the bodies CLConvolution / CLBroadcast / CLBiElementwise /
 *  CLElementwiseFunction / CLScalarBroadcast / CLSum have for OpenCL (KernelCaller.passAllOf(tensor) = data buffer +
 *  inline configuration, KernelCaller.java:41-62), here one downcall each. input(0) is the drain, already on the
 *  device; the drain is returned. COMPILE-UNVERIFIED.
 */
public final class CudaKernels
{
    private static final List<String> FUN_IDS = Arrays.asList(
        "abs", "cbrt", "cos", "exp", "gasu", "gatu", "gaus", "fast_gaus", "gelu", "idy", "log10", "ln",
        "quad", "relu", "selu", "silu", "sig", "sin", "softplus", "softsign", "sqrt", "tanh", "fast_tanh" );

    private CudaKernels() {}

    private static MemorySegment cfg( Arena a, Tensor<?> t ) { return NeurekaCuda.cfg(a, t.getNDConf().asInlineArray()); }

    public static Tensor<?> conv( ExecutionCall<CudaDevice> call, int d ) {
        CudaDevice dev = call.getDevice();
        Tensor<?> t0 = call.input(0), t1 = call.input(1).mut().setIsVirtual(false), t2 = call.input(2).mut().setIsVirtual(false);
        try ( Arena a = Arena.ofConfined() ) {
            NeurekaCuda.check((int) NeurekaCuda.CONV.invokeExact(dev.ctx, CudaDevice.typeOf(t0.getItemType()), t0.rank(),
                    dev.bufOf(t0), cfg(a, t0), dev.bufOf(t1), cfg(a, t1), dev.bufOf(t2), cfg(a, t2), d), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return t0;
    }

    private static Tensor<?> three( java.lang.invoke.MethodHandle h, int op, ExecutionCall<CudaDevice> call, int d ) {
        CudaDevice dev = call.getDevice();
        Tensor<?> t0 = call.input(0).mut().setIsVirtual(false), t1 = call.input(1).mut().setIsVirtual(false), t2 = call.input(2).mut().setIsVirtual(false);
        try ( Arena a = Arena.ofConfined() ) {
            NeurekaCuda.check((int) h.invokeExact(dev.ctx, op, CudaDevice.typeOf(t0.getItemType()), t0.rank(),
                    dev.bufOf(t0), cfg(a, t0), dev.bufOf(t1), cfg(a, t1), dev.bufOf(t2), cfg(a, t2), d), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return t0;
    }

    public static Tensor<?> broadcast( int op, ExecutionCall<CudaDevice> call, int d ) { return three(NeurekaCuda.BROADCAST, op, call, d); }
    public static Tensor<?> binary( int op, ExecutionCall<CudaDevice> call, int d ) { return three(NeurekaCuda.BINARY, op, call, d); }

    public static Tensor<?> scalarBinary( int op, ExecutionCall<CudaDevice> call, int d ) {
        CudaDevice dev = call.getDevice();
        int offset = call.arity() == 3 ? 1 : 0;   // CPUScalarBroadcast.java:32
        Tensor<?> t0 = call.input(0), src = call.input(offset).mut().setIsVirtual(false);
        double value = ((Number) call.input(Number.class, 1 + offset).at(0).get()).doubleValue();
        try ( Arena a = Arena.ofConfined() ) {
            NeurekaCuda.check((int) NeurekaCuda.SCALAR_BIN.invokeExact(dev.ctx, op, CudaDevice.typeOf(t0.getItemType()), t0.rank(),
                    dev.bufOf(t0), cfg(a, t0), dev.bufOf(src), cfg(a, src), value, d), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return t0;
    }

    public static Tensor<?> unary( String funId, ExecutionCall<CudaDevice> call, int d ) {
        CudaDevice dev = call.getDevice();
        Tensor<?> t0 = call.input(0), t1 = call.input(1).mut().setIsVirtual(false);
        try ( Arena a = Arena.ofConfined() ) {
            NeurekaCuda.check((int) NeurekaCuda.UNARY.invokeExact(dev.ctx, FUN_IDS.indexOf(funId), CudaDevice.typeOf(t0.getItemType()), t0.rank(),
                    dev.bufOf(t0), cfg(a, t0), dev.bufOf(t1), cfg(a, t1), d), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return t0;
    }

    public static Tensor<?> fillFun( String funId, ExecutionCall<CudaDevice> call, int d ) {
        CudaDevice dev = call.getDevice();
        Tensor<?> t0 = call.input(0);
        double value = ((Number) call.input(Number.class, 1).at(0).get()).doubleValue();
        try ( Arena a = Arena.ofConfined() ) {
            NeurekaCuda.check((int) NeurekaCuda.FILL_FUN.invokeExact(dev.ctx, FUN_IDS.indexOf(funId), CudaDevice.typeOf(t0.getItemType()), t0.rank(),
                    dev.bufOf(t0), cfg(a, t0), value, d), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return t0;
    }

    public static Tensor<?> sum( ExecutionCall<CudaDevice> call ) {
        CudaDevice dev = call.getDevice();
        Tensor<?> in = call.input(0) == null ? call.input(1) : call.input(0);
        in.mut().setIsVirtual(false);
        Tensor<?> out = Tensor.of(in.getItemType(), neureka.Shape.of(1), 0).mut().setIsVirtual(false);
        dev.store((Tensor<Number>) out);
        try ( Arena a = Arena.ofConfined() ) {
            NeurekaCuda.check((int) NeurekaCuda.SUM.invokeExact(dev.ctx, CudaDevice.typeOf(in.getItemType()), in.rank(),
                    dev.bufOf(in), cfg(a, in), dev.bufOf(out), 0L), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return out;
    }
}
