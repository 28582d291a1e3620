// Minimal JNI declarations for building the Java_* export shim without a JDK.
//
// Only what the shim touches is declared.  JNIEnv is, per the JNI specification, a
// pointer to a pointer to a table of function pointers; the table indices used below
// are the ones the specification's "Interface Function Table" assigns:
//     FindClass 6, Throw 13, NewObjectA 30, GetMethodID 33, NewStringUTF 167, NewIntArray 179,
//     GetLongArrayRegion 204, GetFloatArrayRegion 205, SetIntArrayRegion 211, SetFloatArrayRegion 213.
// When a JDK is present, compile jni_exports.cpp with -DDRAGON_USE_SYSTEM_JNI and the
// JDK's include directories instead; the exported symbols are identical.
#pragma once
#include <stdint.h>

extern "C" {

typedef int32_t jint;
typedef float jfloat;
typedef int64_t jlong;
typedef uint8_t jboolean;
typedef void* jobject;
typedef jobject jclass;
typedef jobject jthrowable;
typedef jobject jarray;
typedef jarray jlongArray;
typedef jarray jintArray;
typedef jarray jfloatArray;
typedef jobject jstring;
typedef void* jmethodID;
typedef union jvalue_ {
  jboolean z; int8_t b; uint16_t c; int16_t s; jint i; jlong j; float f; double d; jobject l;
} jvalue;

typedef const struct JNINativeInterface_min* JNIEnv;

struct JNINativeInterface_min {
  void* slot[230];
};

#define JNIEXPORT __attribute__((visibility("default")))
#define JNICALL

static inline jclass jni_FindClass(JNIEnv* env, const char* name) {
  typedef jclass (*Fn)(JNIEnv*, const char*);
  return reinterpret_cast<Fn>((*env)->slot[6])(env, name);
}
static inline jint jni_Throw(JNIEnv* env, jthrowable obj) {
  typedef jint (*Fn)(JNIEnv*, jthrowable);
  return reinterpret_cast<Fn>((*env)->slot[13])(env, obj);
}
static inline jobject jni_NewObjectA(JNIEnv* env, jclass cls, jmethodID ctor, const jvalue* args) {
  typedef jobject (*Fn)(JNIEnv*, jclass, jmethodID, const jvalue*);
  return reinterpret_cast<Fn>((*env)->slot[30])(env, cls, ctor, args);
}
static inline jmethodID jni_GetMethodID(JNIEnv* env, jclass cls, const char* name, const char* sig) {
  typedef jmethodID (*Fn)(JNIEnv*, jclass, const char*, const char*);
  return reinterpret_cast<Fn>((*env)->slot[33])(env, cls, name, sig);
}
static inline void jni_GetLongArrayRegion(JNIEnv* env, jlongArray arr, jint start, jint len, jlong* buf) {
  typedef void (*Fn)(JNIEnv*, jlongArray, jint, jint, jlong*);
  reinterpret_cast<Fn>((*env)->slot[204])(env, arr, start, len, buf);
}

static inline jstring jni_NewStringUTF(JNIEnv* env, const char* utf) {
  typedef jstring (*Fn)(JNIEnv*, const char*);
  return reinterpret_cast<Fn>((*env)->slot[167])(env, utf);
}
static inline jintArray jni_NewIntArray(JNIEnv* env, jint len) {
  typedef jintArray (*Fn)(JNIEnv*, jint);
  return reinterpret_cast<Fn>((*env)->slot[179])(env, len);
}
static inline void jni_GetFloatArrayRegion(JNIEnv* env, jfloatArray arr, jint start, jint len, jfloat* buf) {
  typedef void (*Fn)(JNIEnv*, jfloatArray, jint, jint, jfloat*);
  reinterpret_cast<Fn>((*env)->slot[205])(env, arr, start, len, buf);
}
static inline void jni_SetIntArrayRegion(JNIEnv* env, jintArray arr, jint start, jint len, const jint* buf) {
  typedef void (*Fn)(JNIEnv*, jintArray, jint, jint, const jint*);
  reinterpret_cast<Fn>((*env)->slot[211])(env, arr, start, len, buf);
}
static inline void jni_SetFloatArrayRegion(JNIEnv* env, jfloatArray arr, jint start, jint len, const jfloat* buf) {
  typedef void (*Fn)(JNIEnv*, jfloatArray, jint, jint, const jfloat*);
  reinterpret_cast<Fn>((*env)->slot[213])(env, arr, start, len, buf);
}

}  // extern "C"
