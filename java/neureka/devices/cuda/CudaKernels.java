package neureka.devices.cuda;

import neureka.Tensor;
import neureka.backend.api.ExecutionCall;

import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;
import java.lang.foreign.ValueLayout;
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

    // ---- fused elementwise expressions (nk_fused_*) ----------------------------------------------------------------------

    private static final java.util.Map<String, MemorySegment> FUSED = new java.util.concurrent.ConcurrentHashMap<>();

    /** Function tree -> "f_tanh(op_add(op_mul(x0,x1),x1))"; n-ary chains nest to the left like reducePairwise. */
    static String fusedExpressionOf( neureka.math.Function f ) {
        if ( f instanceof neureka.math.implementations.FunctionInput ) return "x" + ((neureka.math.implementations.FunctionInput) f).index();
        if ( f instanceof neureka.math.implementations.FunctionConstant ) return "T(" + ((neureka.math.implementations.FunctionConstant) f).value() + ")";
        String id = f.getOperation().getIdentifier();
        java.util.List<neureka.math.Function> subs = f.getSubFunctions();
        String op = switch ( id ) {
            case "add" -> "op_add"; case "subtract" -> "op_sub"; case "multiply" -> "op_mul";
            case "divide" -> "op_div"; case "modulo" -> "op_mod"; case "power" -> "op_pow";
            default -> null;
        };
        if ( op != null ) {
            String acc = fusedExpressionOf( subs.get(0) );
            for ( int i = 1; i < subs.size(); i++ ) acc = op + "(" + acc + ", " + fusedExpressionOf( subs.get(i) ) + ")";
            return acc;
        }
        if ( subs.size() == 1 && f.getOperation() instanceof neureka.backend.main.operations.functions.AbstractActivationOperation )
            return "f_" + id + "(" + fusedExpressionOf( subs.get(0) ) + ")";
        throw new IllegalArgumentException("Operation '" + id + "' is not elementwise and cannot be fused");
    }

    /** Allocates the broadcast-shaped output on the device and launches the compiled kernel once. */
    static Tensor<?> runFused( CudaDevice dev, String expr, int arity, ExecutionCall<?> call ) {
        Tensor<?>[] in = call.inputs();
        int rank = in[0].rank();
        int[] shape = new int[rank];
        for ( int k = 0; k < rank; k++ ) { shape[k] = 1; for ( Tensor<?> t : in ) if ( t.shape(k) != 1 ) shape[k] = t.shape(k); }
        Tensor<?> out = Tensor.of( in[0].getItemType(), neureka.Shape.of(shape), 0 ).mut().setIsIntermediate(true);
        out.mut().setIsVirtual(false);
        dev.store( (Tensor) out );
        int type = CudaDevice.typeOf( in[0].getItemType() );
        try ( Arena a = Arena.ofConfined() ) {
            MemorySegment handle = FUSED.computeIfAbsent( type + ":" + arity + ":" + expr, key -> {
                try ( Arena b = Arena.ofConfined() ) {
                    MemorySegment slot = b.allocate(ValueLayout.ADDRESS);
                    NeurekaCuda.check((int) NeurekaCuda.FUSED_COMPILE.invokeExact(dev.ctx, type, arity, b.allocateFrom(expr), slot), dev.ctx);
                    return slot.get(ValueLayout.ADDRESS, 0);
                } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
            });
            MemorySegment bufs = a.allocate(ValueLayout.ADDRESS, arity), cfgs = a.allocate(ValueLayout.ADDRESS, arity);
            for ( int j = 0; j < arity; j++ ) {
                bufs.setAtIndex(ValueLayout.ADDRESS, j, dev.bufOf(in[j]));
                cfgs.setAtIndex(ValueLayout.ADDRESS, j, NeurekaCuda.cfg(a, in[j].getNDConf().asInlineArray()));
            }
            NeurekaCuda.check((int) NeurekaCuda.FUSED_RUN.invokeExact(dev.ctx, handle, rank, dev.bufOf(out),
                    NeurekaCuda.cfg(a, out.getNDConf().asInlineArray()), bufs, cfgs), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return out;
    }

    // ---- MatMul on the convolution entry point -----------------------------------------------------------------------------

    /** inline array of a rank-2 configuration with one size-1 axis inserted at position `at` (stride / indicesMap of the
     *  new axis are irrelevant: its only index is 0). */
    private static int[] padded( int[] c, int at ) {
        int[] out = new int[15];
        for ( int v = 0; v < 5; v++ ) {                       // shape | strides | indicesMap | offset | spread
            int pad = ( v == 0 || v == 4 ) ? 1 : ( v == 3 ? 0 : 1 );
            for ( int k = 0, j = 0; k < 3; k++ ) out[ v * 3 + k ] = ( k == at ) ? pad : c[ v * 2 + j++ ];
        }
        // the indicesMap of the padded view must be the row-major strides of its shape
        out[8] = 1; out[7] = out[2]; out[6] = out[1] * out[2];
        return out;
    }

    static Tensor<?> matMul( ExecutionCall<CudaDevice> call ) {
        CudaDevice dev = call.getDevice();
        Tensor<?> c = call.input(0), a = call.input(1), b = call.input(2);
        try ( Arena arena = Arena.ofConfined() ) {
            NeurekaCuda.check((int) NeurekaCuda.CONV.invokeExact(dev.ctx, CudaDevice.typeOf(c.getItemType()), 3,
                    dev.bufOf(c), NeurekaCuda.cfg(arena, padded(c.getNDConf().asInlineArray(), 1)),
                    dev.bufOf(a), NeurekaCuda.cfg(arena, padded(a.getNDConf().asInlineArray(), 2)),
                    dev.bufOf(b), NeurekaCuda.cfg(arena, padded(b.getNDConf().asInlineArray(), 0)), -1), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return c;
    }

    // ---- entry points added after the first glue: Min / Max, fused backward, several GPUs in one JVM ----------------------

    /**
     *  Min / Max as the reference's CLReduce / CPUReduce deliver it (operations/other/internal/CPUReduce.java:72-140): the flat
     *  index of the extreme element, lowest index among equals, as a Tensor&lt;Integer&gt; of one item living on the device.
     */
    static Tensor<Integer> argReduce( CudaDevice dev, Tensor<?> in, boolean max ) {
        Tensor<Integer> out = Tensor.of( Integer.class, neureka.Shape.of(1), 0 ).mut().setIsIntermediate(true);
        out.mut().setIsVirtual(false);
        dev.store( out );
        try ( Arena a = Arena.ofConfined() ) {
            NeurekaCuda.check((int) NeurekaCuda.ARG_REDUCE.invokeExact(dev.ctx, max ? 1 : 0, CudaDevice.typeOf(in.getItemType()), in.rank(),
                    dev.bufOf(in), NeurekaCuda.cfg(a, in.getNDConf().asInlineArray()), dev.bufOf(out), 0L), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return out;
    }

    /**
     *  Backward of a fused expression w.r.t. input `target`: one kernel recomputes the expression, multiplies `error`
     *  through it and sums over the dims `target` is broadcast along. `terms` is the statement list of the reverse pass
     *  ("term[0] = ...; ..." over x0..x5 and e, one term per occurrence of the target) -- built from the Function tree the way
     *  neureka_b200/functions.py:fused_gradient_terms_of does; its Java twin is not written yet.
     */
    static Tensor<?> runFusedGrad( CudaDevice dev, String terms, int leaves, int target, Tensor<?> error, Tensor<?>[] in ) {
        int rank = in[0].rank(), arity = in.length;
        Tensor<?> grad = Tensor.of( in[target].getItemType(), in[target].shape(), 0 ).mut().setIsIntermediate(true);
        grad.mut().setIsVirtual(false);
        dev.store( (Tensor) grad );
        int type = CudaDevice.typeOf( in[target].getItemType() );
        try ( Arena a = Arena.ofConfined() ) {
            MemorySegment handle = FUSED.computeIfAbsent( "grad:" + type + ":" + arity + ":" + target + ":" + terms, key -> {
                try ( Arena b = Arena.ofConfined() ) {
                    MemorySegment slot = b.allocate(ValueLayout.ADDRESS);
                    NeurekaCuda.check((int) NeurekaCuda.FUSED_COMPILE_GRAD.invokeExact(dev.ctx, type, arity, target, leaves, b.allocateFrom(terms), slot), dev.ctx);
                    return slot.get(ValueLayout.ADDRESS, 0);
                } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
            });
            MemorySegment bufs = a.allocate(ValueLayout.ADDRESS, arity), cfgs = a.allocate(ValueLayout.ADDRESS, arity);
            for ( int j = 0; j < arity; j++ ) {
                bufs.setAtIndex(ValueLayout.ADDRESS, j, dev.bufOf(in[j]));
                cfgs.setAtIndex(ValueLayout.ADDRESS, j, NeurekaCuda.cfg(a, in[j].getNDConf().asInlineArray()));
            }
            NeurekaCuda.check((int) NeurekaCuda.FUSED_RUN_GRAD.invokeExact(dev.ctx, handle, rank,
                    dev.bufOf(grad), NeurekaCuda.cfg(a, grad.getNDConf().asInlineArray()),
                    dev.bufOf(error), NeurekaCuda.cfg(a, error.getNDConf().asInlineArray()), bufs, cfgs), dev.ctx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
        return grad;
    }

    /**
     *  Forward convolution cut along output dim `dim` over the members of a device group (nk_group_open): slabs[g] / kernels[g]
     *  are the native buffers of member g's input slab and kernel copy, `out` the full result on the first member's device.
     *  The slab extents come from nk_group_plan_slabs (NeurekaCuda.GROUP_PLAN).
     */
    static void convSharded( MemorySegment group, MemorySegment firstCtx, int type, long[] imageShape, long[] kernelShape, int dim,
                             MemorySegment[] slabs, MemorySegment[] kernels, MemorySegment out ) {
        try ( Arena a = Arena.ofConfined() ) {
            MemorySegment sl = a.allocate(ValueLayout.ADDRESS, slabs.length), kl = a.allocate(ValueLayout.ADDRESS, kernels.length);
            for ( int g = 0; g < slabs.length; g++ ) { sl.setAtIndex(ValueLayout.ADDRESS, g, slabs[g]); kl.setAtIndex(ValueLayout.ADDRESS, g, kernels[g]); }
            NeurekaCuda.check((int) NeurekaCuda.CONV_SHARDED.invokeExact(group, type, imageShape.length,
                    a.allocateFrom(ValueLayout.JAVA_LONG, imageShape), a.allocateFrom(ValueLayout.JAVA_LONG, kernelShape), dim, sl, kl, out), firstCtx);
        } catch ( RuntimeException e ) { throw e; } catch ( Throwable t ) { throw new IllegalStateException(t); }
    }
}
